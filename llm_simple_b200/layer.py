"""ctypes binding of the host layer (include/gpu_layer.h): the device memory
pool and the attention section of the transformer layers as Python objects.
Pure plumbing over libgpu_ops.so; nothing is computed here."""
import ctypes

import numpy as np

from . import ops

EXPORTS = [
    "gpu_allocator_allocate", "gpu_allocator_deallocate", "gpu_allocator_stats", "gpu_allocator_trim",
    "gpu_allocator_set_limit", "gpu_allocator_use_host_backend", "gpu_init_freq_cis",
    "gpu_attention_layer_create", "gpu_attention_layer_destroy", "gpu_attention_layer_forward",
    "gpu_attention_layer_decode_ragged", "gpu_attention_layer_set_shared_lens",
    "gpu_attention_layer_forward_host", "gpu_attention_layer_forward_fused", "gpu_attention_layer_cache",
    "gpu_decode_step_create", "gpu_decode_step_destroy", "gpu_decode_step_prepare",
    "gpu_attention_layer_set_shared_step", "gpu_kv_cache_layout", "gpu_attention_layer_set_host_copy_overlap",
]

LLAMA2, QWEN2 = 0, 1
TOKEN_MAJOR, HEAD_MAJOR = 0, 1
_ready = False


def lib():
    global _ready
    L = ops.lib()
    if not _ready:
        vp, i, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t
        L.gpu_allocator_allocate.restype = vp
        L.gpu_allocator_allocate.argtypes = [sz]
        L.gpu_allocator_deallocate.argtypes = [vp]
        L.gpu_allocator_stats.argtypes = [ctypes.POINTER(sz)]
        L.gpu_allocator_set_limit.argtypes = [sz]
        L.gpu_allocator_use_host_backend.argtypes = [i]
        L.gpu_init_freq_cis.argtypes = [vp, i, i, ctypes.c_float, i]
        L.gpu_attention_layer_create.restype = vp
        L.gpu_attention_layer_create.argtypes = [i] * 7 + [ctypes.c_float, i, i, vp, vp, vp]
        L.gpu_attention_layer_destroy.argtypes = [vp]
        L.gpu_attention_layer_forward.argtypes = [vp] * 5 + [i, i, i, vp]
        L.gpu_attention_layer_decode_ragged.argtypes = [vp] * 6 + [i, vp]
        L.gpu_attention_layer_set_shared_lens.argtypes = [vp, vp, i, ctypes.c_long]
        L.gpu_attention_layer_forward_host.argtypes = [vp, vp, vp, i, i, i, vp, vp]
        L.gpu_attention_layer_forward_fused.argtypes = [vp, vp, vp, vp, i, i, i, vp, vp]
        L.gpu_attention_layer_cache.argtypes = [vp, ctypes.POINTER(vp), ctypes.POINTER(vp)]
        L.gpu_decode_step_create.restype = vp
        L.gpu_decode_step_create.argtypes = [i, i, i, i]
        L.gpu_decode_step_destroy.argtypes = [vp]
        L.gpu_decode_step_prepare.argtypes = [vp, vp, i, i, vp]
        L.gpu_attention_layer_set_shared_step.argtypes = [vp, vp]
        L.gpu_attention_layer_set_host_copy_overlap.argtypes = [vp, i]
        L.gpu_kv_cache_layout.restype = sz
        L.gpu_kv_cache_layout.argtypes = [ctypes.POINTER(ops.AttnDesc), i, i, i, i]
        _ready = True
    return L


def allocator_stats():
    out = (ctypes.c_size_t * 5)()
    lib().gpu_allocator_stats(out)
    return dict(zip(["backend_bytes", "pooled_bytes", "backend_allocs", "pool_hits", "backend_frees"],
                    [int(x) for x in out]))


def init_freq_cis(head_dim, max_seq_len, theta, dt):
    out = np.empty((max_seq_len, head_dim // 2, 2), dtype=np.float32)
    lib().gpu_init_freq_cis(out.ctypes.data, head_dim, max_seq_len, theta, dt)
    return out


def kv_cache_layout(desc, cache_layout, n_kv_heads, max_seq_len, head_dim=128):
    """Fills desc's three cache strides for the layout; returns the elements per sequence."""
    return int(lib().gpu_kv_cache_layout(ctypes.byref(desc), cache_layout, n_kv_heads, max_seq_len, head_dim))


class DecodeStep:
    """Per-step state a model shares between its layers: the work partition of the decode
    step for the sequences' cache lengths, uploaded once (gpu_decode_step_*)."""

    def __init__(self, max_batch, n_heads, n_kv_heads, dt):
        self.h = lib().gpu_decode_step_create(max_batch, n_heads, n_kv_heads, dt)
        if not self.h:
            raise ops.GpuOpsError("gpu_decode_step_create failed")

    def prepare(self, kv_len, append_new=True, stream=None):
        lens = np.ascontiguousarray(kv_len, dtype=np.int32)
        ops._check(lib().gpu_decode_step_prepare(self.h, lens.ctypes.data, len(lens), int(bool(append_new)),
                                                 ops._stream(stream)))

    def close(self):
        if self.h:
            lib().gpu_decode_step_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class AttentionLayer:
    """Handle of one layer's attention section (Llama-2 or Qwen2 flavour)."""

    def __init__(self, kind, n_heads, n_kv_heads, max_seq_len, max_batch, dt, rope_theta, rope_is_neox_style,
                 cache_layout=HEAD_MAJOR, shared_freq_cis=None, k_cache=None, v_cache=None, head_dim=128):
        self._keep = (shared_freq_cis, k_cache, v_cache)
        self.h = lib().gpu_attention_layer_create(
            kind, n_heads, n_kv_heads, head_dim, max_seq_len, max_batch, dt, rope_theta,
            int(bool(rope_is_neox_style)), cache_layout, ops._ptr(shared_freq_cis), ops._ptr(k_cache),
            ops._ptr(v_cache))
        if not self.h:
            raise ops.GpuOpsError("gpu_attention_layer_create failed")

    def close(self):
        if self.h:
            lib().gpu_attention_layer_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def forward(self, out, q, k, v, batch, cur_pos, prev_pos, stream=None):
        ops._check(lib().gpu_attention_layer_forward(self.h, ops._ptr(out), ops._ptr(q), ops._ptr(k), ops._ptr(v),
                                                     batch, cur_pos, prev_pos, ops._stream(stream)))

    def decode_ragged(self, out, q, k, v, kv_len, stream=None):
        lens = np.ascontiguousarray(kv_len, dtype=np.int32)
        ops._check(lib().gpu_attention_layer_decode_ragged(self.h, ops._ptr(out), ops._ptr(q), ops._ptr(k),
                                                           ops._ptr(v), lens.ctypes.data, len(lens),
                                                           ops._stream(stream)))

    def set_shared_lens(self, kv_len_dev, max_kv_len, total_kv_len=0):
        ops._check(lib().gpu_attention_layer_set_shared_lens(self.h, ops._ptr(kv_len_dev), max_kv_len,
                                                             total_kv_len))

    def set_shared_step(self, step):
        """step: a DecodeStep prepared for this decode step, or None."""
        self._step = step
        ops._check(lib().gpu_attention_layer_set_shared_step(self.h, step.h if step is not None else None))

    def set_host_copy_overlap(self, on):
        """False: forward_host copies its input on the caller's stream, behind that stream's earlier
        work; True (the default): on the layer's own stream, the caller's stream waits for it."""
        ops._check(lib().gpu_attention_layer_set_host_copy_overlap(self.h, int(bool(on))))

    def forward_host(self, out_host, qkv_host, batch, cur_pos, prev_pos, kv_len=None, stream=None):
        lens_ptr = None
        if kv_len is not None:
            lens = np.ascontiguousarray(kv_len, dtype=np.int32)
            lens_ptr = lens.ctypes.data
        ops._check(lib().gpu_attention_layer_forward_host(self.h, ops._ptr(out_host), ops._ptr(qkv_host), batch,
                                                          cur_pos, prev_pos, lens_ptr, ops._stream(stream)))

    def forward_fused(self, out, qkv, bias, batch, cur_pos, prev_pos, kv_len=None, stream=None):
        """Device tensors: qkv [batch][cur_size][(H + 2 kvH)*D], bias one such row or None."""
        lens_ptr = None
        if kv_len is not None:
            lens = np.ascontiguousarray(kv_len, dtype=np.int32)
            lens_ptr = lens.ctypes.data
        ops._check(lib().gpu_attention_layer_forward_fused(self.h, ops._ptr(out), ops._ptr(qkv), ops._ptr(bias), batch,
                                                           cur_pos, prev_pos, lens_ptr, ops._stream(stream)))

    def cache_ptrs(self):
        k, v = ctypes.c_void_p(), ctypes.c_void_p()
        ops._check(lib().gpu_attention_layer_cache(self.h, ctypes.byref(k), ctypes.byref(v)))
        return k.value, v.value
