// Compiles the C++ host mirror against the C ABI and exercises its host-only parts (no GPU needed):
// PagedKvTable known answers (src/paged_kv.rs:200-270), layouts, typed errors, no-device behaviour.
#include <cstdio>
#include <cstdlib>

#include "../flat-attention_b200/host/flat_attention.hpp"

#define CHECK(x)                                                        \
    do {                                                                \
        if (!(x)) {                                                     \
            std::fprintf(stderr, "CHECK failed: %s (line %d)\n", #x, __LINE__); \
            return 1;                                                   \
        }                                                               \
    } while (0)

int main() {
    using namespace flat;
    PagedKvTable t(4, 3);
    t.append(9);
    CHECK(t.address(0)->physical_page == 0);
    CHECK(t.address(3)->offset_in_page == 3);
    CHECK(t.address(4)->physical_page == 1);
    CHECK(t.address(8)->physical_page == 2);
    CHECK(!t.address(9).has_value());
    bool threw = false;
    try {
        t.append(4);
    } catch (const Error &e) {
        threw = e.status() == FLAT_ERR_CAPACITY_EXCEEDED;
    }
    CHECK(threw && t.len() == 9);
    t.reset();
    CHECK(t.generation() == 1 && t.is_empty());

    auto shape = AttentionShape::grouped(2, 8, 2, 17, 64);
    auto L = CudaGroupedForwardPipeline::layout(DType::F32, shape);
    CHECK(L.q_elements == 2u * 8 * 17 * 64 && L.lse_byte_offset == 4 * L.q_elements);
    auto BL = CudaGroupedBackwardRecomputePipeline::layout(DType::F32, shape);
    CHECK(BL.k_offset == 4 * BL.q_elements && BL.output_bytes == 4 * (BL.q_elements + 2 * BL.kv_elements));
    threw = false;
    try {
        forward_layout(DType::F32, AttentionShape::grouped(1, 6, 4, 2, 8));
    } catch (const Error &e) {
        threw = e.status() == FLAT_ERR_INVALID_HEAD_GROUPING;
    }
    CHECK(threw);
    FlatAttentionConfig cfg;
    CHECK(cfg.raw().has_softmax_scale == 0);
    cfg.softmax_scale = 0.25f;
    CHECK(cfg.raw().has_softmax_scale == 1 && cfg.raw().softmax_scale == 0.25f);
    // telemetry records and manifests are host-only (src/runtime_telemetry.rs:207-214, src/benchmark_manifest.rs:285-316)
    flat_device_fingerprint fp{};
    std::snprintf(fp.name, sizeof fp.name, "GPU a;b=c%%");
    std::snprintf(fp.backend, sizeof fp.backend, "Cuda");
    fp.vendor = 0x10de;
    fp.device = 100;
    CHECK(canonical_record(fp) == "name=GPU a%3bb%3dc%25;backend=Cuda;driver=;driver_info=;vendor=000010de;device=00000064");
    CHECK(stable_fingerprint(fp) == stable_fingerprint(fp));
    flat_benchmark_manifest m{};
    m.commit_sha = "main";
    threw = false;
    try {
        canonical_json(m);
    } catch (const Error &e) {
        threw = e.status() == FLAT_ERR_MANIFEST_INVALID_COMMIT_SHA;
    }
    CHECK(threw);
    // routing table and numerical guarantees are pure (src/wgpu_f16_backend.rs:491-497, src/numerical.rs:68-96)
    CHECK(CudaPreferredAttention::io_precision_for_head_dim(64) == FLAT_IO_PACKED_F16);
    CHECK(CudaPreferredAttention::io_precision_for_head_dim(80) == FLAT_IO_F32);
    CHECK(NumericalExecutor::guarantees(FLAT_NUMERICAL_DETERMINISTIC_PORTABLE).repeatable_same_backend_device == 1);
    CHECK(NumericalExecutor::guarantees(FLAT_NUMERICAL_FAST_PORTABLE).allows_subgroup == 1);
    CHECK(forward_layout(DType::F16, shape).q_bytes == 2 * L.q_elements);
    // without an sm_100 device a context cannot be created, and nothing falls back to the CPU
    if (std::getenv("FLAT_EXPECT_NO_DEVICE")) {
        threw = false;
        try {
            Context ctx(0);
        } catch (const Error &e) {
            threw = e.status() == FLAT_ERR_UNAVAILABLE;
        }
        CHECK(threw);
    }
    std::puts("host mirror ok");
    return 0;
}
