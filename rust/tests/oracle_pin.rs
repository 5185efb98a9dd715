//! Pins the C++ restatement of the scalar oracle (oracle/flat_oracle.cpp, the checker of every CUDA parity test) to
//! the reference's own Rust oracle: the same seeded inputs through both, every output compared BITWISE.
//!
//!     cargo test --features oracle-pin --test oracle_pin
//!
//! Needs no GPU.  It is the one artefact that can close the "parity unpinned" gap: the machines this backend was
//! built on have no Rust toolchain, so the restatement has so far been checked against the reference's oracle-only
//! tests restated in Python, not against executed reference output.
#![cfg(feature = "oracle-pin")]

use flat_attention::{
    backward_reference_grouped, forward_reference, forward_reference_grouped, forward_reference_grouped_rope, AttentionShape,
    FlatAttentionConfig, GroupedAttentionShape, RotaryEmbeddingConfig,
};
use flat_attention_cuda::cuda_types::{FlatAttentionConfigRaw, FlatAttentionShape};

extern "C" {
    fn flat_oracle_forward_reference(q: *const f32, q_n: u64, k: *const f32, k_n: u64, v: *const f32, v_n: u64, batch: u64,
                                     heads: u64, seq_len: u64, head_dim: u64, cfg: *const FlatAttentionConfigRaw, out: *mut f32,
                                     lse: *mut f32) -> i32;
    fn flat_oracle_forward_grouped_asymmetric(q: *const f32, q_n: u64, k: *const f32, k_n: u64, v: *const f32, v_n: u64,
                                              shape: *const FlatAttentionShape, cfg: *const FlatAttentionConfigRaw, out: *mut f32,
                                              lse: *mut f32) -> i32;
    fn flat_oracle_forward_grouped_rope(q: *const f32, q_n: u64, k: *const f32, k_n: u64, v: *const f32, v_n: u64,
                                        shape: *const FlatAttentionShape, cfg: *const FlatAttentionConfigRaw, theta: f32,
                                        position_offset: u64, out: *mut f32, lse: *mut f32) -> i32;
    fn flat_oracle_backward_grouped(q: *const f32, q_n: u64, k: *const f32, k_n: u64, v: *const f32, v_n: u64, d_out: *const f32,
                                    d_out_n: u64, fwd_out: *const f32, fwd_out_n: u64, fwd_lse: *const f32, fwd_lse_n: u64,
                                    batch: u64, q_heads: u64, kv_heads: u64, seq_len: u64, head_dim: u64,
                                    cfg: *const FlatAttentionConfigRaw, dq: *mut f32, dk: *mut f32, dv: *mut f32) -> i32;
}

/// splitmix64 -> uniform -> Box-Muller N(0, 1), the generator the benchmark fixtures use.
fn normal(n: usize, seed: u64) -> Vec<f32> {
    let mut state = seed;
    let mut next = || {
        state = state.wrapping_add(0x9E37_79B9_7F4A_7C15);
        let mut z = state;
        z = (z ^ (z >> 30)).wrapping_mul(0xBF58_476D_1CE4_E5B9);
        z = (z ^ (z >> 27)).wrapping_mul(0x94D0_49BB_1331_11EB);
        z ^ (z >> 31)
    };
    let mut out = Vec::with_capacity(n);
    while out.len() < n {
        let u1 = ((next() >> 11) as f64 + 1.0) / 9_007_199_254_740_993.0;
        let u2 = (next() >> 11) as f64 / 9_007_199_254_740_992.0;
        let r = (-2.0 * u1.ln()).sqrt();
        out.push((r * (2.0 * std::f64::consts::PI * u2).cos()) as f32);
        out.push((r * (2.0 * std::f64::consts::PI * u2).sin()) as f32);
    }
    out.truncate(n);
    out
}

fn bits(v: &[f32]) -> Vec<u32> {
    v.iter().map(|x| x.to_bits()).collect()
}

fn raw(c: FlatAttentionConfig) -> FlatAttentionConfigRaw {
    FlatAttentionConfigRaw { causal: c.causal as i32, has_softmax_scale: c.softmax_scale.is_some() as i32,
                             softmax_scale: c.softmax_scale.unwrap_or(0.0) }
}

#[test]
fn forward_reference_is_bitwise_identical() {
    // the reference's own CPU-runnable configuration: MHA, causal, [1, 2, 128, 64]
    for &(b, h, n, d, causal) in &[(1usize, 2usize, 128usize, 64usize, true), (2, 3, 37, 20, false), (1, 1, 1, 2, true)] {
        let len = b * h * n * d;
        let (q, k, v) = (normal(len, 1), normal(len, 2), normal(len, 3));
        let cfg = FlatAttentionConfig { causal, softmax_scale: None };
        let want = forward_reference(&q, &k, &v, AttentionShape { batch: b, heads: h, seq_len: n, head_dim: d }, cfg).unwrap();
        let (mut o, mut l) = (vec![0f32; len], vec![0f32; b * h * n]);
        let st = unsafe {
            flat_oracle_forward_reference(q.as_ptr(), len as u64, k.as_ptr(), len as u64, v.as_ptr(), len as u64, b as u64, h as u64,
                                          n as u64, d as u64, &raw(cfg), o.as_mut_ptr(), l.as_mut_ptr())
        };
        assert_eq!(st, 0);
        assert_eq!(bits(&o), bits(&want.output));
        assert_eq!(bits(&l), bits(&want.lse));
    }
}

#[test]
fn grouped_and_rotary_forward_are_bitwise_identical() {
    for &(b, hq, hkv, n, d, causal, scale) in &[(1usize, 8usize, 2usize, 67usize, 32usize, true, None), (2, 4, 4, 19, 16, false, Some(0.3f32)),
                                                 (1, 6, 1, 33, 64, true, None)] {
        let (ql, kl) = (b * hq * n * d, b * hkv * n * d);
        let (q, k, v) = (normal(ql, 11), normal(kl, 12), normal(kl, 13));
        let cfg = FlatAttentionConfig { causal, softmax_scale: scale };
        let shape = GroupedAttentionShape { batch: b, q_heads: hq, kv_heads: hkv, seq_len: n, head_dim: d };
        let raw_shape = FlatAttentionShape { batch: b as u64, q_heads: hq as u64, kv_heads: hkv as u64, query_len: n as u64,
                                             kv_len: n as u64, head_dim: d as u64, query_position_offset: 0 };
        let want = forward_reference_grouped(&q, &k, &v, shape, cfg).unwrap();
        let (mut o, mut l) = (vec![0f32; ql], vec![0f32; b * hq * n]);
        assert_eq!(unsafe {
            flat_oracle_forward_grouped_asymmetric(q.as_ptr(), ql as u64, k.as_ptr(), kl as u64, v.as_ptr(), kl as u64, &raw_shape,
                                                   &raw(cfg), o.as_mut_ptr(), l.as_mut_ptr())
        }, 0);
        assert_eq!(bits(&o), bits(&want.output));
        assert_eq!(bits(&l), bits(&want.lse));

        let rotary = RotaryEmbeddingConfig { theta: 500_000.0, position_offset: 4090 };
        let want = forward_reference_grouped_rope(&q, &k, &v, shape, cfg, rotary).unwrap();
        assert_eq!(unsafe {
            flat_oracle_forward_grouped_rope(q.as_ptr(), ql as u64, k.as_ptr(), kl as u64, v.as_ptr(), kl as u64, &raw_shape, &raw(cfg),
                                             rotary.theta, rotary.position_offset as u64, o.as_mut_ptr(), l.as_mut_ptr())
        }, 0);
        assert_eq!(bits(&o), bits(&want.output));
        assert_eq!(bits(&l), bits(&want.lse));
    }
}

#[test]
fn grouped_backward_is_bitwise_identical() {
    for &(b, hq, hkv, n, d, causal) in &[(1usize, 4usize, 2usize, 23usize, 16usize, true), (2, 2, 2, 9, 8, false)] {
        let (ql, kl) = (b * hq * n * d, b * hkv * n * d);
        let (q, k, v, d_out) = (normal(ql, 21), normal(kl, 22), normal(kl, 23), normal(ql, 24));
        let cfg = FlatAttentionConfig { causal, softmax_scale: None };
        let shape = GroupedAttentionShape { batch: b, q_heads: hq, kv_heads: hkv, seq_len: n, head_dim: d };
        let fwd = forward_reference_grouped(&q, &k, &v, shape, cfg).unwrap();
        let want = backward_reference_grouped(&q, &k, &v, &d_out, shape, cfg, &fwd).unwrap();
        let (mut dq, mut dk, mut dv) = (vec![0f32; ql], vec![0f32; kl], vec![0f32; kl]);
        assert_eq!(unsafe {
            flat_oracle_backward_grouped(q.as_ptr(), ql as u64, k.as_ptr(), kl as u64, v.as_ptr(), kl as u64, d_out.as_ptr(), ql as u64,
                                         fwd.output.as_ptr(), ql as u64, fwd.lse.as_ptr(), (b * hq * n) as u64, b as u64, hq as u64,
                                         hkv as u64, n as u64, d as u64, &raw(cfg), dq.as_mut_ptr(), dk.as_mut_ptr(), dv.as_mut_ptr())
        }, 0);
        assert_eq!(bits(&dq), bits(&want.dq));
        assert_eq!(bits(&dk), bits(&want.dk));
        assert_eq!(bits(&dv), bits(&want.dv));
    }
}
