"""Regenerates the golden fixtures in this directory from the reference checkout.

Run where the reference tree is mounted:  python tests/golden/make_golden.py /path/to/reference
The fixtures are committed; tests never read the reference tree.

Two convolution example graphs ship with the reference (examples/test_conv2d_1x1_1x32x32x8_*), each with the
input tensor and the output TensorFlow Lite produced; the reference's own unit test compares its fp32 result with
that output (reference_model/test/model_runner_tests.cpp:85-125).  The constant operands live inside the
serialized .tosa graphs.  No flatbuffer schema is available, so the constants are taken from fixed byte offsets
that were located by matching: the fp32 weights are the 512-byte block equal to the least-squares solution of
output = input x W; the int8 weights are the 128-byte block whose products correlate (r = 0.9999) with the output;
the RESCALE multipliers / shifts are the only run of sixteen int32 values in [2^30, 2^31) / sixteen int8 values
of 40.  The quantized graph's bias (0), input zero point (0) and output zero point (-2) are the unique small
values for which CONV2D + per-channel DOUBLE_ROUND RESCALE reproduces all 16384 expected outputs exactly
(SINGLE_ROUND differs in 11 of them), so this fixture pins the double-rounding rule.
"""
import os
import sys

import numpy as np


def main(ref_root):
    here = os.path.dirname(os.path.abspath(__file__))
    ex = os.path.join(ref_root, "examples")

    d = os.path.join(ex, "test_conv2d_1x1_1x32x32x8_f32_st11_padSAME_dilat11")
    raw = open(os.path.join(d, "flatbuffer-tflite", "test_conv2d_1x1_1x32x32x8_f32_st11_padSAME_dilat11.tosa"),
               "rb").read()
    w = np.frombuffer(raw[396:396 + 512], dtype=np.float32).reshape(16, 1, 1, 8)
    np.savez_compressed(os.path.join(here, "conv2d_1x1_f32_example.npz"),
                        x=np.load(os.path.join(d, "placeholder_0.npy")), w=w, bias=np.zeros(16, np.float32),
                        expected=np.load(os.path.join(d, "tflite_result.npy")))

    d = os.path.join(ex, "test_conv2d_1x1_1x32x32x8_qi8_st11_padSAME_dilat11")
    raw = open(os.path.join(d, "flatbuffer-tflite", "test_conv2d_1x1_1x32x32x8_qi8_st11_padSAME_dilat11.tosa"),
               "rb").read()
    np.savez_compressed(os.path.join(here, "conv2d_1x1_qi8_example.npz"),
                        x=np.load(os.path.join(d, "placeholder_0.npy")),
                        w=np.frombuffer(raw[484:484 + 128], dtype=np.int8).reshape(16, 1, 1, 8),
                        bias=np.zeros(16, np.int32),
                        multiplier=np.frombuffer(raw[808:808 + 64], dtype=np.int32),
                        shift=np.frombuffer(raw[928:928 + 16], dtype=np.int8),
                        input_zp=np.int32(0), weight_zp=np.int32(0), output_zp=np.int32(-2),
                        expected=np.load(os.path.join(d, "tflite_result.npy")))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the TOSA reference model>")
    main(sys.argv[1])
