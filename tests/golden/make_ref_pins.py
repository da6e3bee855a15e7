"""Writes tests/golden/ref_pins.npz from REFERENCE CODE compiled here (oracle/build_ref.py ->
oracle/_ref/libref_pins.so): known-answer vectors of the pieces of the hot path that the
reference holds as plain C++.  Needs the reference tree; the fixture travels without it.

    python tests/golden/make_ref_pins.py

  bf16_in / bf16_out      fp32_to_bfloat16 (src/util.cpp:33-72) on edge patterns and seeded random ones
  table_*                 rows of ModelBase::InitFreqCIS (src/model_base.cpp:27-83) incl. position 32 767+
  rope_*_in / _gold       the golden loop of tests/rope_single_layer_test.cpp:78-97 on seeded 16-bit
                          inputs, rounded to the type with torch (the test rounds with Eigen's cast)
  mask                    the mask loop of tests/flash_attn_test.cpp:124-132
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import ref_pins as ref  # noqa: E402

FP16, BF16 = 4, 5


def to_bits_and_back(x, dt):
    import torch
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.float16 if dt == FP16 else torch.bfloat16)
    return t.view(torch.int16).numpy().view(np.uint16), t.to(torch.float32).numpy()


def main():
    if not ref.available():
        raise SystemExit("the reference tree is needed to write this fixture")
    out = {}
    rng = np.random.default_rng(20250)
    edge = [0x00000000, 0x80000000, 0x3f800000, 0x3f808000, 0x3f818000, 0x3f80ffff, 0x3f7fffff, 0x7f7fffff, 0x7f800000,
            0xff800000, 0x00000001, 0x007fffff, 0x00800000, 0x3effffff, 0xbf7f8000, 0x3f7f8000, 0x3f7f7fff, 0x477fe000]
    pats = np.concatenate([np.array(edge, dtype=np.uint32), rng.integers(0, 1 << 32, size=4096, dtype=np.uint64).astype(np.uint32)])
    out["bf16_in"] = pats
    out["bf16_out"] = np.array([ref.fp32_to_bfloat16(int(u)) for u in pats], dtype=np.uint16)
    rows = np.array([0, 1, 2, 3, 7, 255, 511, 766, 2047, 2303, 4096, 8191, 32767, 32768, 32895], dtype=np.int64)
    out["table_rows"] = rows
    out["table_1e4_fp16"] = ref.model_init_freq_cis(128, 32896, 1e4, FP16)[rows]
    out["table_1e6_bf16"] = ref.model_init_freq_cis(128, 32896, 1e6, BF16)[rows]
    offset, heads, seq = 509, 3, 5
    out["rope_offset"], out["rope_heads"] = np.int32(offset), np.int32(heads)
    for dt, dname in ((FP16, "fp16"), (BF16, "bf16")):
        table = ref.model_init_freq_cis(128, offset + seq, 1e6 if dt == BF16 else 1e4, dt)
        x_bits, x32 = to_bits_and_back(rng.standard_normal((seq, heads * 128), dtype=np.float32), dt)
        for neox, nname in ((False, "inter"), (True, "neox")):
            gold32 = ref.rope_golden(x32, table, offset, heads, 128, neox)
            out["rope_%s_%s_in" % (dname, nname)] = x_bits
            out["rope_%s_%s_gold" % (dname, nname)] = to_bits_and_back(gold32, dt)[1]
    out["mask_shape"] = np.array([7, 20, 12], dtype=np.int32)
    out["mask"] = ref.causal_mask(7, 20, 12)
    path = os.path.join(ROOT, "tests", "golden", "ref_pins.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
