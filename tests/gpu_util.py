"""Helpers shared by the GPU parity tests: moving raw 16-bit patterns between
numpy (what the oracle takes) and torch CUDA tensors (what the C ABI is handed),
and the parity rule."""
import numpy as np
import torch

from oracle import oracle as orc

FP16, BF16 = orc.DT_FLOAT16, orc.DT_BFLOAT16
TORCH_DT = {FP16: torch.float16, BF16: torch.bfloat16}
D = 128

# north-star tolerance for fp16 / bf16 attention with fp32 accumulation
MAX_ABS = 1e-2
MEAN_ABS = 1e-3


def dev(bits, dt):
    """numpy uint16 bit patterns -> CUDA tensor of the 16-bit dtype (same shape)."""
    t = torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).cuda()
    return t.view(TORCH_DT[dt])


def host(t):
    """CUDA 16-bit tensor -> numpy uint16 bit patterns."""
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def rnd_bits(shape, dt, seed):
    rng = np.random.default_rng(seed)
    return orc.to_bits(rng.standard_normal(shape, dtype=np.float32), dt)


def ulp(x, dt):
    """Spacing of the 16-bit dtype at magnitude |x| (normal range)."""
    mant = 10 if dt == FP16 else 7
    e = np.floor(np.log2(np.maximum(np.abs(x), 2.0 ** -14)))
    return np.exp2(e - mant)


def parity(out_bits, golden_f32, dt):
    """Compare a 16-bit GPU result with an fp32 golden.

    The golden is rounded to the dtype first (the reference's own tests do the
    same, tests/rope_single_layer_test.cpp:97).  Returns (max_abs, mean_abs, ok).
    ok: mean_abs <= 1e-3 and every element within max(1e-2, one ulp of the dtype
    at that magnitude) -- bf16 has 8 significant bits, so where |x| >= 2 two
    neighbouring representable values are already 1.6e-2 apart and a correctly
    rounded result of a differently ordered sum may land on the neighbour.
    """
    out = orc.to_f32(out_bits, dt).ravel()
    gold = orc.to_f32(orc.to_bits(golden_f32, dt), dt).ravel()
    diff = np.abs(out - gold)
    allowed = np.maximum(MAX_ABS, ulp(gold, dt))
    ok = bool(np.all(np.isfinite(out)) and diff.mean() <= MEAN_ABS and np.all(diff <= allowed))
    return float(diff.max()), float(diff.mean()), ok


def assert_parity(out_bits, golden_f32, dt, what=""):
    mx, mean, ok = parity(out_bits, golden_f32, dt)
    assert ok, "%s: max_abs %.3e mean_abs %.3e" % (what, mx, mean)
    return mx, mean
