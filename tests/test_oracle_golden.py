"""The CPU oracle (oracle/e8_oracle.c) against fixtures produced by the unmodified reference.

These tests are what pins the oracle: every function it restates must reproduce the reference's
float32 output bit for bit on the committed golden vectors (tests/golden/make_golden.py).
"""
import numpy as np
import pytest

from conftest import bits
from oracle import oracle as O


def test_generators(golden_codec):
    g, gi = O.generators()
    assert np.array_equal(g, golden_codec["G"])
    assert np.array_equal(gi, golden_codec["Ginv"])


def test_custom_round_known_answers(golden_codec):
    # the reference's own test pins custom_round(+-0.5) == 0 (tests/legacy/test_lattices.py:113-123)
    assert O.custom_round(np.array([0.5, -0.5], np.float32)).tolist() == [0.0, 0.0]
    got = O.custom_round(golden_codec["cr_in"])
    assert np.array_equal(bits(got), bits(golden_codec["cr_out"]))


def test_projection_and_gx(golden_codec):
    x = golden_codec["proj_in"]
    assert np.array_equal(bits(O.projection(x)), bits(golden_codec["proj_out"]))
    assert np.array_equal(bits(O.g_x(x)), bits(golden_codec["gx_out"]))


@pytest.mark.parametrize("name,s", [("s0p25", 0.25), ("s0p5", 0.5), ("s1", 1.0), ("s2", 2.0), ("s4", 4.0), ("s8", 8.0)])
def test_encode_decode_scale_sweep(golden_codec, name, s):
    x = golden_codec["cfg1_x"] * np.float32(s)
    codes = O.encode(x)
    assert np.array_equal(O.codes_to_int(codes), golden_codec[f"cfg1_codesA_{name}"].astype(np.int64))
    assert np.array_equal(bits(O.decode(codes)), bits(golden_codec[f"cfg1_xhatA_{name}"]))


def test_literal_layer_convention_is_all_zero(golden_codec):
    beta = np.float32(0.021440971642732620)
    codes = O.encode(golden_codec["cfg1_x"], beta=beta, scale_mode=2, blocks_per_tile=1 << 40)
    assert not codes.any()
    assert not golden_codec["cfg1_codesA_lit"].any()
    xh = O.decode(codes, beta=beta, scale_mode=2, blocks_per_tile=1 << 40)
    assert np.array_equal(bits(xh), bits(golden_codec["cfg1_xhatA_lit"]))


@pytest.mark.parametrize("name,b", [("mid", 0.021440971642732620), ("0p3", 0.3), ("1p7", 1.7)])
def test_codec_convention(golden_codec, name, b):
    codes = O.encode(golden_codec["cfg1_x"], beta=b, scale_mode=1)
    assert np.array_equal(O.codes_to_int(codes), golden_codec[f"cfg1_codesB_{name}"].astype(np.int64))
    xh = O.decode(codes, beta=b, scale_mode=1)
    assert np.array_equal(bits(xh), bits(golden_codec[f"cfg1_xhatB_{name}"]))


@pytest.mark.parametrize("q,M", [(2, 1), (3, 2), (4, 1), (4, 3), (5, 2), (8, 2), (16, 2)])
def test_other_q_m(golden_codec, q, M):
    x = golden_codec["cfg1_x"][:2048] * np.float32(3.0)
    codes = O.encode(x, beta=0.7, scale_mode=1, q=q, M=M)
    assert np.array_equal(O.codes_to_int(codes), golden_codec[f"qm_codes_{q}_{M}"].astype(np.int64))
    xh = O.decode(codes, beta=0.7, scale_mode=1, q=q)
    assert np.array_equal(bits(xh), bits(golden_codec[f"qm_xhat_{q}_{M}"]))


def test_adversarial_rows(golden_codec):
    x = golden_codec["adv_x"]
    codes = O.encode(x)
    assert np.array_equal(O.codes_to_int(codes), golden_codec["adv_codes"].astype(np.int64))
    assert np.array_equal(bits(O.decode(codes)), bits(golden_codec["adv_xhat"]))
    assert np.array_equal(bits(O.quantize(x)), bits(golden_codec["adv_quant"]))


def test_quantize(golden_codec):
    x = golden_codec["cfg1_x"]
    assert np.array_equal(bits(O.quantize(x)), bits(golden_codec["cfg1_quant_s1"]))
    assert np.array_equal(bits(O.quantize(x * np.float32(4.0))), bits(golden_codec["cfg1_quant_s4"]))


def test_exhaustive_single_level_decode(golden_decode_table):
    idx = np.arange(65536)
    digits = np.stack([(idx >> (2 * j)) & 3 for j in range(8)], axis=1).astype(np.float32)
    res = O.decode(digits[:, None, :])
    assert np.array_equal((res * 2).astype(np.int8), golden_decode_table)
    assert len(np.unique(golden_decode_table, axis=0)) == 65536
    assert golden_decode_table.min() == -7 and golden_decode_table.max() == 11


@pytest.mark.parametrize("tag", ["small", "big", "mid"])
def test_layer_fake_quant(golden_layer, tag):
    W = golden_layer[f"{tag}_W"]
    o, i = W.shape
    wq, _ = O.fake_quant(W.reshape(-1, 8), golden_layer[f"{tag}_beta"], i // 8)
    assert np.array_equal(bits(wq.reshape(o, i)), bits(golden_layer[f"{tag}_Wq"]))
    wqb, _ = O.fake_quant(W.reshape(-1, 8), golden_layer[f"{tag}_blk_beta"].reshape(-1), 1)
    assert np.array_equal(bits(wqb.reshape(o, i)), bits(golden_layer[f"{tag}_blk_Wq"]))
