"""The CPU oracle against the reference's own known-answer tests and example graphs.

Every case below restates a case of the reference's unit tests; the file:line of the original is given.
"""
import os

import numpy as np
import pytest

from oracle import oracle as orc

# reference_model/test/ref_model_tests/tensor_ops_tests.cpp:622-683 (inVals, weightVals, inZp, weightZp)
ZP_CASES = [
    ([126, -126, -120, 0], [2, 1, 4, -7], 4, 15),        # :628-631 input negative overflow
    ([122, -7, -120, 121], [2, 1, 4, -7], -10, -5),      # :643-646 input positive overflow
    ([3, -12, 5, 70], [-120, -12, 0, -7], 55, 15),       # :658-661 weight negative overflow
    ([-5, 65, -1, 32], [-2, 125, 4, -1], -10, -5),       # :673-676 weight positive overflow
]


def _expected_dot(inv, wv, izp, wzp):
    # tensor_ops_tests.cpp:102-107
    return sum((int(a) - izp) * (int(b) - wzp) for a, b in zip(inv, wv))


@pytest.mark.parametrize("inv,wv,izp,wzp", ZP_CASES)
def test_conv2d_zero_point_kat(inv, wv, izp, wzp):
    # testConv2d, tensor_ops_tests.cpp:72-121: 1x2x2x1 input, 1x2x2x1 weight, stride 2, one output
    x = np.array(inv, np.int8).reshape(1, 2, 2, 1)
    w = np.array(wv, np.int8).reshape(1, 2, 2, 1)
    out = orc.conv2d(x, w, np.zeros(1, np.int32), [0, 0, 0, 0], [2, 2], [1, 1], izp, wzp)
    assert out.shape == (1, 1, 1, 1)
    assert int(out[0, 0, 0, 0]) == _expected_dot(inv, wv, izp, wzp)


@pytest.mark.parametrize("inv,wv,izp,wzp", ZP_CASES)
def test_depthwise_zero_point_kat(inv, wv, izp, wzp):
    # testDepthwiseConv2d, tensor_ops_tests.cpp:170-219: weight [2,2,1,1]
    x = np.array(inv, np.int8).reshape(1, 2, 2, 1)
    w = np.array(wv, np.int8).reshape(2, 2, 1, 1)
    out = orc.depthwise_conv2d(x, w, np.zeros(1, np.int32), [0, 0, 0, 0], [2, 2], [1, 1], izp, wzp)
    assert int(out[0, 0, 0, 0]) == _expected_dot(inv, wv, izp, wzp)


@pytest.mark.parametrize("av,bv,azp,bzp", ZP_CASES)
def test_matmul_zero_point_kat(av, bv, azp, bzp):
    # testMatMul, tensor_ops_tests.cpp:448-506: A [1,2,2], B [1,2,2]
    a = np.array(av, np.int8).reshape(1, 2, 2)
    b = np.array(bv, np.int8).reshape(1, 2, 2)
    exp = (a.astype(np.int64) - azp)[0] @ (b.astype(np.int64) - bzp)[0]
    out = orc.matmul(a, b, azp, bzp)
    assert np.array_equal(out[0], exp)


def test_conv2d_bias_broadcast_kat():
    # tensor_ops_tests.cpp:736-766 with testConv2dBias :124-168: input [1,1,1,2], weight [2,1,1,2]
    x = np.array([5, 9], np.int8).reshape(1, 1, 1, 2)
    w = np.array([3, -7, -1, 4], np.int8).reshape(2, 1, 1, 2)
    out = orc.conv2d(x, w, np.array([-5], np.int32), [0, 0, 0, 0], [1, 1], [1, 1])
    assert out.reshape(-1).tolist() == [5 * 3 + 9 * (-7) + (-5), 5 * (-1) + 9 * 4 + (-5)]
    out = orc.conv2d(x, w, np.array([-5, 14], np.int32), [0, 0, 0, 0], [1, 1], [1, 1])
    assert out.reshape(-1).tolist() == [5 * 3 + 9 * (-7) + (-5), 5 * (-1) + 9 * 4 + 14]


def test_depthwise_bias_broadcast_kat():
    # tensor_ops_tests.cpp:768-798: input [1,1,1,2], weight [1,1,2,1]
    x = np.array([5, 9], np.int8).reshape(1, 1, 1, 2)
    w = np.array([3, -7], np.int8).reshape(1, 1, 2, 1)
    out = orc.depthwise_conv2d(x, w, np.array([-5], np.int32), [0, 0, 0, 0], [1, 1], [1, 1])
    assert out.reshape(-1).tolist() == [5 * 3 + (-5), 9 * (-7) + (-5)]
    out = orc.depthwise_conv2d(x, w, np.array([-5, 14], np.int32), [0, 0, 0, 0], [1, 1], [1, 1])
    assert out.reshape(-1).tolist() == [5 * 3 + (-5), 9 * (-7) + 14]


@pytest.mark.parametrize("inv,izp,ozp", [([126, -126, -128, 0], 4, 15), ([126, 126, 127, 127], -12, -5)])
def test_avg_pool2d_zero_point_kat(inv, izp, ozp):
    # tensor_ops_tests.cpp:800-822, expectation formula :552-564
    x = np.array(inv, np.int8).reshape(1, 2, 2, 1)
    s = sum(int(v) - izp for v in inv)
    res = (s * ((1 << 30) + 1) + (1 << 31)) >> 32
    exp = min(max(res + ozp, -128), 127)
    st, out = orc.avg_pool2d(x, [2, 2], [0, 0, 0, 0], [2, 2], izp, ozp)
    assert st == orc.VALID and int(out[0, 0, 0, 0]) == exp


def test_rescale_output_zp_extension_kat():
    # type_conversion_tests.cpp:324-335: i8 -> u16, scale16, (((65 - 1) * 4 + (1 << 1)) >> 2) + 32768 = 32832
    st, out = orc.rescale(np.array([65]), [4], [2], per_channel=False, scale32=False, rounding="SINGLE_ROUND",
                          input_zp=1, output_zp=32768, in_bits=8, out_bits=16, output_unsigned=True)
    assert st == orc.VALID and out.tolist() == [32832]


def test_rescale_inexact_round_kat():
    # type_conversion_tests.cpp:385-404
    st, out = orc.rescale(np.array([65]), [4], [2], per_channel=False, scale32=False, rounding="INEXACT_ROUND",
                          input_zp=1, output_zp=32768, in_bits=8, out_bits=16, output_unsigned=True)
    assert st == orc.VALID and out.tolist() == [32832]
    st, out = orc.rescale(np.array([103]), [147], [8], per_channel=False, scale32=False, rounding="INEXACT_ROUND",
                          input_zp=-95, output_zp=0, in_bits=8, out_bits=8, output_unsigned=True)
    assert st == orc.VALID and out.tolist() == [114]


@pytest.mark.parametrize("mult,shift,per_channel,scale32,in_bits,out_bits,vals", [
    ([4, 2], [16, 5, 9], True, True, 8, 32, [20, -5, -16]),        # :337-347 size(multiplier) != NC
    ([4, 1024, 2048, 115], [12], True, False, 32, 8, [0, -12, 0, 12]),  # :349-359 size(shift) != NC
    ([4, 519], [12], False, True, 8, 32, [20, -5, -16]),           # :361-371 per_channel=false, 2 multipliers
    ([4], [6, 16], False, False, 32, 8, [0, -12, 0, 12]),          # :373-383 per_channel=false, 2 shifts
])
def test_rescale_operand_size_errors_kat(mult, shift, per_channel, scale32, in_bits, out_bits, vals):
    st, _ = orc.rescale(np.array(vals), mult, shift, per_channel=per_channel, scale32=scale32, in_bits=in_bits,
                        out_bits=out_bits)
    assert st == orc.ERROR


def test_apply_scale_32_hand_derived():
    # quant_util.h:45-84, worked by hand: double rounding adds +-2^30 before the shift only when shift > 31
    assert orc.apply_scale_32(1, 1 << 30, 31, True) == (True, 1)      # (2^30 + 2^30) >> 31 = 1
    assert orc.apply_scale_32(1, 1 << 30, 32, False) == (True, 0)     # (2^30 + 2^31) >> 32 = 0
    assert orc.apply_scale_32(1, 1 << 30, 32, True) == (True, 1)      # (2^30 + 2^31 + 2^30) >> 32 = 1
    assert orc.apply_scale_32(-1, 1 << 30, 32, True) == (True, 0)     # (-2^30 + 2^31 - 2^30) >> 32 = 0
    assert orc.apply_scale_32(-3, 1 << 30, 32, False) == (True, -1)   # (-3*2^30 + 2^31) >> 32 = floor(-0.25) = -1
    assert orc.apply_scale_32(-3, 1 << 30, 32, True) == (True, -1)    # (-3*2^30 + 2^31 - 2^30) >> 32 = floor(-.5)
    assert orc.apply_scale_32((1 << 29), 1 << 30, 30, True)[0] is False   # value >= 2^(shift-1) violates the range
    assert orc.apply_scale_32(5, -1, 30, True)[0] is False
    assert orc.apply_scale_32(5, 7, 1, True)[0] is False
    assert orc.apply_scale_32(5, 7, 63, True)[0] is False


def test_reciprocal_scale():
    # quant_util.h:32-43: count 4 -> k = 2, multiplier ((2^30+1) << 2) / 4, shift 32; count 49 -> k = 6
    assert orc.reciprocal_scale(4) == ((1 << 30) + 1, 32)
    assert orc.reciprocal_scale(49) == ((((1 << 30) + 1) << 6) // 49, 36)
    assert orc.reciprocal_scale(1) == ((1 << 30) + 1, 30)


def test_conv2d_fp32_example_graph(golden_dir):
    # reference_model/test/model_runner_tests.cpp:85-125 runs examples/test_conv2d_1x1_1x32x32x8_f32_* and compares
    # with the TensorFlow Lite output using doctest::Approx (relative epsilon 1e-5 scaled)
    g = np.load(os.path.join(golden_dir, "conv2d_1x1_f32_example.npz"))
    out = orc.conv2d(g["x"], g["w"], g["bias"], [0, 0, 0, 0], [1, 1], [1, 1], mode="f32")
    assert out.shape == g["expected"].shape
    np.testing.assert_allclose(out, g["expected"], rtol=1e-4, atol=1e-5)


def test_conv2d_qi8_example_graph(golden_dir):
    # examples/test_conv2d_1x1_1x32x32x8_qi8_*: CONV2D + per-channel RESCALE (shift 40, DOUBLE_ROUND)
    g = np.load(os.path.join(golden_dir, "conv2d_1x1_qi8_example.npz"))
    acc = orc.conv2d(g["x"], g["w"], g["bias"], [0, 0, 0, 0], [1, 1], [1, 1], int(g["input_zp"]),
                     int(g["weight_zp"]))
    st, out = orc.rescale(acc, g["multiplier"], g["shift"], per_channel=True, scale32=True,
                          rounding="DOUBLE_ROUND", input_zp=0, output_zp=int(g["output_zp"]), in_bits=32,
                          out_bits=8)
    assert st == orc.VALID
    assert np.array_equal(out, g["expected"].astype(np.int32))
    st, single = orc.rescale(acc, g["multiplier"], g["shift"], per_channel=True, scale32=True,
                             rounding="SINGLE_ROUND", input_zp=0, output_zp=int(g["output_zp"]), in_bits=32,
                             out_bits=8)
    assert int((single != g["expected"]).sum()) == 11


def test_conv_attribute_rules():
    # tensor_ops.cpp:203-223: exact-division rule; a 7x7 stride-2 pad-3 stem on 224 is illegal, pad [3,2,3,2] is legal
    assert orc.check_conv2d_attribute(224, 224, 112, 112, 7, 7, [3, 3, 3, 3], [2, 2], [1, 1]) == 4
    assert orc.check_conv2d_attribute(224, 224, 112, 112, 7, 7, [3, 2, 3, 2], [2, 2], [1, 1]) == 0
    assert orc.check_conv2d_attribute(56, 56, 56, 56, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1]) == 0
    assert orc.check_conv2d_attribute(56, 56, 55, 56, 3, 3, [1, 1, 1, 1], [1, 1], [1, 1]) == 5
    assert orc.check_conv2d_attribute(8, 8, 8, 8, 3, 3, [-1, 1, 1, 1], [1, 1], [1, 1]) == 1
    assert orc.check_conv2d_attribute(8, 8, 8, 8, 3, 3, [1, 1, 1, 1], [0, 1], [1, 1]) == 2
    assert orc.check_conv2d_attribute(8, 8, 8, 8, 3, 3, [1, 1, 1, 1], [1, 1], [1, 0]) == 3
    # tensor_ops.cpp:94-114
    assert orc.check_pool2d_attribute(112, 112, 56, 56, [3, 3], [1, 0, 1, 0], [2, 2]) == 0
    assert orc.check_pool2d_attribute(112, 112, 56, 56, [3, 3], [1, 1, 1, 1], [2, 2]) == 5
    assert orc.check_pool2d_attribute(8, 8, 8, 8, [2, 2], [2, 0, 0, 0], [1, 1]) == 4


def test_fp_rounding_helpers():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(7)
    v = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-8, 5, 4096),
                        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 6e-8, 2.0 ** -24, 2.0 ** -25,
                                  3 * 2.0 ** -25, np.inf, -np.inf], np.float32)])
    t = torch.from_numpy(v)
    assert np.array_equal(orc.fptrunc(v, "fp16"), t.to(torch.float16).float().numpy())
    assert np.array_equal(orc.fptrunc(v, "bf16"), t.to(torch.bfloat16).float().numpy())


def test_clamp_and_add_semantics():
    st, out = orc.clamp(np.array([-200, -128, 0, 127, 300]), -100, 100)
    assert st == orc.VALID and out.tolist() == [-100, -100, 0, 100, 100]
    assert orc.clamp(np.array([1]), 5, 4)[0] == orc.ERROR       # activation_funcs.cpp:97
    st, out = orc.clamp(np.array([np.nan, 7.0, -1.0], np.float32), 0.0, 6.0, mode="f32", fdt="fp16")
    assert np.isnan(out[0]) and out[1:].tolist() == [6.0, 0.0]
    st, out = orc.clamp(np.array([np.nan], np.float32), 0.0, 6.0, mode="f32", nan_ignore=True)
    assert out.tolist() == [0.0]
    st, out = orc.add(np.array([[1, 2], [3, 4]]), np.array([[10], [20]]))
    assert st == orc.VALID and out.tolist() == [[11, 12], [23, 24]]
    st, out = orc.add(np.array([2147483647]), np.array([1]))
    assert st == orc.UNPREDICTABLE and out.tolist() == [-2147483648]
    assert orc.add(np.zeros((2, 3)), np.zeros((2, 2)))[0] == orc.ERROR
    st, out = orc.add(np.array([1.0009765625], np.float32), np.array([2.0 ** -12], np.float32), mode="f32", fdt="fp16")
    assert out.tolist() == [1.0009765625]   # 1 + 2^-10 + 2^-12 rounds back to 1 + 2^-10 in binary16


def test_max_pool_padding_value():
    x = np.full((1, 2, 2, 1), -128, np.int8)
    out = orc.max_pool2d(x, [3, 3], [1, 1, 1, 1], [1, 1])   # (2+2-3)/1+1 = 2
    assert out.shape == (1, 2, 2, 1) and (out == -128).all()
    x = np.arange(16, dtype=np.int8).reshape(1, 4, 4, 1)
    out = orc.max_pool2d(x, [2, 2], [0, 0, 0, 0], [2, 2])
    assert out.reshape(-1).tolist() == [5, 7, 13, 15]


def test_precise_and_bounds_modes_and_verifier():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 6, 6, 8)).astype(np.float32)
    w = rng.standard_normal((4, 3, 3, 8)).astype(np.float32)
    b = rng.standard_normal(4).astype(np.float32)
    args = ([1, 1, 1, 1], [1, 1], [1, 1])
    normal = orc.conv2d(x, w, b, *args, mode="f32")
    ref = orc.conv2d(x, w, b, *args, mode="f64")
    bnd = orc.conv2d(x, w, b, *args, mode="f64", bounds=True)
    assert (bnd >= np.abs(ref) - 1e-12).all()
    ksb = orc.dot_product_ksb(3 * 3 * 8 + 1)
    ok, info = orc.verify_dot_product(normal, ref, bnd, ksb)
    assert ok and info["max_abs_err"] < 2 * ksb
    ok, _ = orc.verify_dot_product(normal + 1e-2, ref, bnd, ksb)
    assert not ok
    # multi-threaded split must not change a single bit
    assert np.array_equal(orc.conv2d(x, w, b, *args, mode="f32", nthreads=4), normal)


# --------------------------------------------------------------------------------------------- TRANSPOSE_CONV2D
def _spread_and_mirror(x, w, out_pad, stride, fill):
    """The CONV2D that equals a TRANSPOSE_CONV2D: input spread by the stride, kernel mirrored, pads K-1+out_pad."""
    N, IH, IW, IC = x.shape
    _, KH, KW, _ = w.shape
    d = np.full((N, (IH - 1) * stride[0] + 1, (IW - 1) * stride[1] + 1, IC), fill, x.dtype)
    d[:, ::stride[0], ::stride[1], :] = x
    pad = [KH - 1 + out_pad[0], KH - 1 + out_pad[1], KW - 1 + out_pad[2], KW - 1 + out_pad[3]]
    return d, np.ascontiguousarray(w[:, ::-1, ::-1, :]), pad


def test_transpose_conv2d_hand_case():
    # one row [1, 2], kernel [3, 4], stride 2: every input pixel stamps the kernel, no overlap
    x = np.array([1, 2], np.int8).reshape(1, 1, 2, 1)
    w = np.array([3, 4], np.int8).reshape(1, 1, 2, 1)
    out = orc.transpose_conv2d(x, w, np.array([10], np.int32), [0, 0, 0, 0], [1, 2])
    assert out.reshape(-1).tolist() == [13, 14, 16, 18]
    # stride 1: the stamps overlap and add; out_pad_left = -1 drops the first column, out_pad_right = 1 adds an empty one
    out = orc.transpose_conv2d(x, w, np.array([0], np.int32), [0, 0, 0, 0], [1, 1])
    assert out.reshape(-1).tolist() == [3, 4 + 6, 8]
    out = orc.transpose_conv2d(x, w, np.array([0], np.int32), [0, 0, -1, 1], [1, 1])
    assert out.reshape(-1).tolist() == [10, 8, 0]
    # zero points are subtracted from both operands (tensor_ops.cpp:2163-2168)
    out = orc.transpose_conv2d(x, w, np.array([0], np.int32), [0, 0, 0, 0], [1, 2], in_zp=1, w_zp=-1)
    assert out.reshape(-1).tolist() == [0, 0, 4, 5]


@pytest.mark.parametrize("shape,out_pad,stride", [
    ((2, 5, 6, 7, 3, 3, 2), (0, 1, -1, 0), (2, 3)),
    ((1, 4, 4, 3, 5, 2, 4), (-1, -1, 2, 1), (1, 1)),
    ((1, 3, 3, 2, 2, 3, 3), (1, 0, 0, 2), (3, 2)),
    ((1, 6, 5, 4, 4, 4, 4), (-3, -3, -3, -3), (2, 2)),
])
def test_transpose_conv2d_equals_conv2d_of_spread_input(shape, out_pad, stride):
    N, IH, IW, IC, OC, KH, KW = shape
    rng = np.random.default_rng(IH * 100 + KW)
    x = rng.integers(-128, 128, (N, IH, IW, IC)).astype(np.int8)
    w = rng.integers(-128, 128, (OC, KH, KW, IC)).astype(np.int8)
    b = rng.integers(-1000, 1000, OC).astype(np.int32)
    got = orc.transpose_conv2d(x, w, b, out_pad, stride, -5, 3)
    assert got.shape[1:3] == orc.transpose_conv_out_hw(IH, IW, KH, KW, out_pad, stride)
    d, wm, pad = _spread_and_mirror(x, w, out_pad, stride, -5)
    assert np.array_equal(got, orc.conv2d(d, wm, b, pad, [1, 1], [1, 1], -5, 3))
    assert np.array_equal(got, orc.transpose_conv2d(x, w, b, out_pad, stride, -5, 3, nthreads=4))
    # precise mode: same sums in doubles, up to the order of the taps
    xf, wf, bf = x.astype(np.float64) / 64, w.astype(np.float64) / 64, b.astype(np.float64) / 64
    d, wm, pad = _spread_and_mirror(xf, wf, out_pad, stride, 0.0)
    assert np.allclose(orc.transpose_conv2d(xf, wf, bf, out_pad, stride, mode="f64"),
                       orc.conv2d(d, wm, bf, pad, [1, 1], [1, 1], mode="f64"), rtol=0, atol=1e-9)


def test_transpose_conv2d_attribute_rules():
    # tensor_ops.cpp:2038-2054: out_pad > -kernel, output size (I-1)*stride + out_pad + K
    assert orc.check_transpose_conv2d_attribute(4, 4, 9, 9, 3, 3, [0, 0, 0, 0], [2, 2]) == 0
    assert orc.check_transpose_conv2d_attribute(4, 4, 9, 9, 3, 3, [0, 0, 0, 0], [0, 2]) != 0
    assert orc.check_transpose_conv2d_attribute(4, 4, 6, 9, 3, 3, [-3, 0, 0, 0], [2, 2]) != 0
    assert orc.check_transpose_conv2d_attribute(4, 4, 7, 9, 3, 3, [-2, 0, 0, 0], [2, 2]) == 0
    assert orc.check_transpose_conv2d_attribute(4, 4, 10, 9, 3, 3, [0, 0, 0, 0], [2, 2]) != 0


def test_fp8_decode_matches_torch_casts():
    import torch
    codes = np.arange(256, dtype=np.uint8)
    for fmt, tdt in (("e4m3", torch.float8_e4m3fn), ("e5m2", torch.float8_e5m2)):
        mine = orc.fp8_to_f32(codes, fmt)
        theirs = torch.from_numpy(codes.copy()).view(tdt).to(torch.float32).numpy()
        assert np.array_equal(np.isnan(mine), np.isnan(theirs))
        ok = ~np.isnan(mine)
        assert np.array_equal(mine[ok], theirs[ok]) and np.array_equal(np.signbit(mine[ok]), np.signbit(theirs[ok]))
    assert orc.fp8_to_f32([0x7E], "e4m3")[0] == 448.0 and orc.fp8_to_f32([0x01], "e4m3")[0] == 2.0 ** -9
    assert orc.fp8_to_f32([0x7B], "e5m2")[0] == 57344.0 and orc.fp8_to_f32([0x01], "e5m2")[0] == 2.0 ** -16


# reference_model/test/ref_model_tests/tensor_ops_tests.cpp:685-735 (inVals, weightVals, inZp, weightZp)
ZP_CASES_3D = [
    ([127, -128, 126, -127, 125, -126, 124, -125], [2, -2, 1, -1, 3, -3, 4, -4], 4, 15),          # :691-696
    ([122, -7, -120, 121, 123, -8, -119, 120], [2, 1, 4, -7, 3, -2, 5, -6], -10, -5),             # :703-708
    ([3, -12, 5, 70, -10, 20, 15, 25], [-120, -12, 0, -7, -50, 10, -30, 5], 55, 15),              # :715-720
    ([-5, 65, -1, 32, 20, -10, -15, 5], [-2, 125, 4, -1, -20, 30, 60, 120], -10, -5),             # :727-732
]


@pytest.mark.parametrize("inv,wv,izp,wzp", ZP_CASES_3D)
def test_conv3d_zero_point_kat(inv, wv, izp, wzp):
    # testConv3d, tensor_ops_tests.cpp:395-445: 1x2x2x2x1 input, 1x2x2x2x1 weight, no padding, stride 1, one output
    x = np.array(inv, np.int8).reshape(1, 2, 2, 2, 1)
    w = np.array(wv, np.int8).reshape(1, 2, 2, 2, 1)
    out = orc.conv3d(x, w, np.zeros(1, np.int32), [0] * 6, [1, 1, 1], [1, 1, 1], izp, wzp)
    assert out.shape == (1, 1, 1, 1, 1)
    assert int(out[0, 0, 0, 0, 0]) == _expected_dot(inv, wv, izp, wzp)


def test_conv3d_against_conv2d_and_numpy():
    """A CONV3D with one depth tap is a CONV2D over the depth slices (the CONV2D restatement is pinned above), and a full
    3-D case agrees with a plain numpy evaluation of the definition (tensor_ops.cpp:1060-1106), padding, strides and
    dilation included."""
    r = np.random.default_rng(11)
    x = r.integers(-128, 128, size=(2, 3, 6, 5, 4), dtype=np.int8)
    w = r.integers(-127, 128, size=(3, 1, 3, 2, 4), dtype=np.int8)
    b = r.integers(-1000, 1000, size=3).astype(np.int32)
    out = orc.conv3d(x, w, b, [0, 0, 1, 1, 0, 1], [1, 2, 1], [1, 1, 2], -3, 5)
    ref = orc.conv2d(x.reshape(6, 6, 5, 4), w.reshape(3, 3, 2, 4), b, [1, 1, 0, 1], [2, 1], [1, 2], -3, 5)
    assert np.array_equal(out.reshape(ref.shape), ref)
    x = r.integers(-128, 128, size=(1, 5, 4, 6, 3), dtype=np.int8)
    w = r.integers(-127, 128, size=(2, 2, 3, 2, 3), dtype=np.int8)
    b = r.integers(-1000, 1000, size=1).astype(np.int32)
    pad, stride, dil, izp, wzp = [1, 1, 1, 1, 0, 2], [2, 1, 2], [2, 1, 3], 7, -2
    out = orc.conv3d(x, w, b, pad, stride, dil, izp, wzp)
    OD, OH, OW = orc.conv3d_out_dhw(5, 4, 6, 2, 3, 2, pad, stride, dil)
    assert orc.check_conv3d_attribute(5, 4, 6, OD, OH, OW, 2, 3, 2, pad, stride, dil) == 0
    assert orc.check_conv3d_attribute(5, 4, 6, OD, OH, OW + 1, 2, 3, 2, pad, stride, dil) == 5
    assert orc.check_conv3d_attribute(5, 4, 7, OD, OH, OW, 2, 3, 2, pad, stride, dil) == 4    # (7 - 1 + 2 - 3) % 2 != 0
    exp = np.zeros((1, OD, OH, OW, 2), np.int64)
    for od in range(OD):
        for oy in range(OH):
            for ox in range(OW):
                for kd in range(2):
                    for ky in range(3):
                        for kx in range(2):
                            d, y, xx = od * 2 + kd * 2 - 1, oy + ky - 1, ox * 2 + kx * 3
                            if 0 <= d < 5 and 0 <= y < 4 and 0 <= xx < 6:
                                exp[0, od, oy, ox] += (x[0, d, y, xx].astype(np.int64) - izp) @ (w[:, kd, ky, kx].astype(np.int64) - wzp).T
    assert np.array_equal(out, exp + int(b[0]))
    # the floating instantiations on the same taps
    xf, wf = x.astype(np.float32) / 16, w.astype(np.float32) / 64
    f32 = orc.conv3d(xf, wf, np.zeros(1, np.float32), pad, stride, dil, mode="f32")
    f64 = orc.conv3d(xf, wf, np.zeros(1), pad, stride, dil, mode="f64")
    np.testing.assert_allclose(f32, f64, rtol=1e-5, atol=1e-5)
    bnd = orc.conv3d(xf, wf, np.zeros(1), pad, stride, dil, mode="f64", bounds=True)
    assert np.all(bnd >= np.abs(f64) - 1e-12)
