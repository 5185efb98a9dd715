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
