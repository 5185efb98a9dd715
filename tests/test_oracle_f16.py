"""Pins of the binary16 conversion restated from src/f16.rs: the reference's unit tests
(src/f16.rs:146-191) and an exhaustive / randomized comparison with numpy's IEEE float16."""
import numpy as np

from oracle import binding as ob


def test_known_binary16_encodings_match_ieee754():
    # src/f16.rs:150-158
    vals = np.array([0.0, -0.0, 1.0, -2.0, 65504.0, np.inf], np.float32)
    assert ob.f16_from_f32(vals).tolist() == [0x0000, 0x8000, 0x3c00, 0xc000, 0x7bff, 0x7c00]


def test_binary16_decoding_handles_normals_and_subnormals():
    # src/f16.rs:160-166
    got = ob.f16_to_f32(np.array([0x3c00, 0xc000, 0x0400, 0x0001], np.uint16))
    assert got.tolist() == [1.0, -2.0, 2.0 ** -14, 2.0 ** -24]


def test_finite_roundtrip_has_binary16_scale_error():
    # src/f16.rs:168-183
    for value in [-17.75, -1.0, -0.33325, 0.0, 0.1, 1.0, np.pi, 1024.5]:
        decoded = float(ob.f16_round([value])[0])
        assert abs(decoded - np.float32(value)) <= 5.0e-4 * max(abs(value), 1.0)


def test_non_finite_classification_is_explicit():
    # src/f16.rs:185-190
    bits = ob.f16_from_f32(np.array([1.0, np.inf, np.nan], np.float32))
    finite = (bits & 0x7c00) != 0x7c00
    assert finite.tolist() == [True, False, False]


def test_decoding_matches_ieee_for_every_bit_pattern():
    bits = np.arange(65536, dtype=np.uint16)
    mine, ieee = ob.f16_to_f32(bits), bits.view(np.float16).astype(np.float32)
    nan = np.isnan(ieee)
    assert np.array_equal(np.isnan(mine), nan)
    assert np.array_equal(mine[~nan].view(np.uint32), ieee[~nan].view(np.uint32))


def test_encoding_matches_ieee_round_to_nearest_even():
    rng = np.random.default_rng(16)
    # random bit patterns cover every exponent; add the rounding boundaries of every binary16 value
    x = rng.integers(0, 2 ** 32, 400000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    h = np.arange(0x7c00, dtype=np.uint16).view(np.float16).astype(np.float64)
    mid = ((h[:-1] + h[1:]) / 2).astype(np.float32)  # exact ties
    edge = np.concatenate([mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf)),
                           np.array([65504.0, 65519.99, 65520.0, 1e-8, 2.0 ** -25, 2.0 ** -24, 3e-8], np.float32)])
    x = np.concatenate([x, edge, -edge])
    keep = ~np.isnan(x)
    with np.errstate(over="ignore"):
        ieee = x[keep].astype(np.float16).view(np.uint16)
    assert np.array_equal(ob.f16_from_f32(x[keep]), ieee)
    nan_bits = ob.f16_from_f32(x[~keep])
    assert ((nan_bits & 0x7c00) == 0x7c00).all() and ((nan_bits & 0x03ff) != 0).all()
