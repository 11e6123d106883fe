"""Regenerates tests/golden/codec_folds.json from the reference's own host codecs.

Needs oracle/_ref/libref_codecs.so (``make -f oracle/Makefile`` with the reference mounted).  For every encoder the fold
is a 64-bit order-independent hash of code(x) over all 2^32 FP32 bit patterns; the CPU test recomputes it from the
oracle's independent encoders, so equality means equality on every input."""
import ctypes
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
ref = ctypes.CDLL(os.path.join(HERE, "..", "..", "oracle", "_ref", "libref_codecs.so"))
ref.ref_encoder_fold.restype = ctypes.c_uint64
ref.ref_encoder_fold.argtypes = [ctypes.c_int, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int]
out = {"_comment": "64-bit folds of code(x) over ALL 2^32 FP32 bit patterns (oracle.encoder_fold), produced by the REFERENCE's own host "
                   "codecs (src/nvfp4effma.cuh:137-210, tests/test_util.h:51 there) through oracle/_ref/libref_codecs.so; regenerate with "
                   "tests/golden/make_codec_folds.py"}
for which, name in enumerate(["e4m3", "e2m1", "ue5m3", "bf16"]):
    out[name] = hex(ref.ref_encoder_fold(which, 0, 1 << 32, os.cpu_count() or 1))
json.dump(out, open(os.path.join(HERE, "codec_folds.json"), "w"), indent=2)
print(out)
