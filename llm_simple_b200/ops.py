"""ctypes binding of libgpu_ops.so: one Python function per C entry point of
include/gpu_ops.h, same names, same argument order.

Tensor arguments are torch CUDA tensors (or raw integer device addresses); the
wrappers pass ``data_ptr()`` through and launch on torch's current stream unless
``stream`` is given.  A non-zero status raises GpuOpsError with the library's
message.  Nothing here computes anything: without the compiled library every
call fails.
"""
import ctypes
import os

DT_FLOAT16 = 4   # reference DataType values (prebuild/defs.hpp:8-18)
DT_BFLOAT16 = 5

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libgpu_ops.so")
_lib = None

EXPORTS = [
    "gpu_flash_attn_layer", "gpu_flash_attn_gqa_layer", "gpu_flash_attn_opt_prefill_layer",
    "gpu_rope_layer", "gpu_rope_single_layer", "gpu_split_qkv_layer", "gpu_rope_kv_append_layer",
    "gpu_qkv_rope_kv_append_layer", "gpu_bias_add_layer", "gpu_attn_prefill_layer",
    "gpu_attn_decode_layer", "gpu_attn_decode_layer_noalloc", "gpu_attn_decode_noalloc_prepare", "gpu_attn_decode_plan_bytes", "gpu_attn_decode_plan",
    "gpu_attn_decode_plan_size", "gpu_attn_decode_plan_workspace_bytes", "gpu_attn_decode_planned_layer", "gpu_rope_kv_append_paged_layer",
    "gpu_attn_decode_paged_layer", "gpu_attn_prefill_paged_layer", "gpu_attn_decode_workspace_bytes", "gpu_attn_merge_lse_layer", "gpu_attn_merge_packed_layer",
    "gpu_attn_xchg_buffer_bytes", "gpu_attn_xchg_local_slot", "gpu_attn_xchg_merge_layer",
    "gpu_attn_decode_xchg_layer",
    "gpu_peer_buffer_alloc", "gpu_peer_buffer_open", "gpu_peer_buffer_close", "gpu_peer_buffer_free",
    "gpu_ops_set_workspace", "gpu_attn_set_decode_chunk", "gpu_attn_set_decode_early_prefetch", "gpu_attn_set_prefill_kernel", "gpu_attn_set_prefill_l2_window", "gpu_attn_last_prefill_kernel",
    "gpu_ops_launch_count", "gpu_ops_last_error_string", "gpu_ops_kernel_status", "gpu_ops_clear_kernel_status",
]


class GpuOpsError(RuntimeError):
    pass


class KvPages(ctypes.Structure):
    """struct gpu_kv_pages (include/gpu_ops.h): page table of a paged KV cache."""
    _fields_ = [("page_table", ctypes.c_void_p), ("table_stride", ctypes.c_int32), ("page_size", ctypes.c_int32),
                ("page_stride", ctypes.c_int64), ("n_pages", ctypes.c_int32), ("reserved", ctypes.c_int32)]


def make_pages(page_table, page_size, page_stride, n_pages):
    """page_table: device int32 tensor [batch][entries]; page_stride in elements; n_pages in the pool."""
    pg = KvPages()
    pg.page_table = _ptr(page_table)
    pg.table_stride = page_table.shape[1]
    pg.page_size = page_size
    pg.page_stride = page_stride
    pg.n_pages = n_pages
    pg._keep = page_table
    return pg


class AttnDesc(ctypes.Structure):
    """struct gpu_attn_desc (include/gpu_ops.h); strides in elements."""
    _fields_ = [
        ("dtype", ctypes.c_int32), ("batch", ctypes.c_int32), ("n_heads", ctypes.c_int32),
        ("n_kv_heads", ctypes.c_int32), ("head_dim", ctypes.c_int32), ("is_neox_style", ctypes.c_int32),
        ("q_seq_stride", ctypes.c_int64), ("q_tok_stride", ctypes.c_int64),
        ("kv_in_seq_stride", ctypes.c_int64), ("kv_in_tok_stride", ctypes.c_int64),
        ("out_seq_stride", ctypes.c_int64), ("out_tok_stride", ctypes.c_int64),
        ("cache_seq_stride", ctypes.c_int64), ("cache_head_stride", ctypes.c_int64),
        ("cache_pos_stride", ctypes.c_int64), ("total_kv_len", ctypes.c_int64),
    ]


def make_desc(dtype, batch, n_heads, n_kv_heads, m, max_pos, layout="head", is_neox=False, head_dim=128):
    """Descriptor for dense q/out [batch][m][H][D], raw k/v [batch][m][kvH][D] and a
    cache of `max_pos` positions per sequence: head-major [batch][kvH][max_pos][D]
    or token-major [batch][max_pos][kvH][D] (the reference's layout)."""
    d = AttnDesc()
    d.dtype, d.batch, d.n_heads, d.n_kv_heads, d.head_dim = dtype, batch, n_heads, n_kv_heads, head_dim
    d.is_neox_style = int(bool(is_neox))
    d.q_tok_stride = n_heads * head_dim
    d.q_seq_stride = m * d.q_tok_stride
    d.out_tok_stride = n_heads * head_dim
    d.out_seq_stride = m * d.out_tok_stride
    d.kv_in_tok_stride = n_kv_heads * head_dim
    d.kv_in_seq_stride = m * d.kv_in_tok_stride
    d.cache_seq_stride = n_kv_heads * max_pos * head_dim
    if layout == "head":
        d.cache_head_stride, d.cache_pos_stride = max_pos * head_dim, head_dim
    elif layout == "token":
        d.cache_head_stride, d.cache_pos_stride = head_dim, n_kv_heads * head_dim
    else:
        raise ValueError(layout)
    return d


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "%s is missing: build it with `python -m llm_simple_b200.build` "
                "(there is no CPU or PyTorch fallback)" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        vp, i, i32p, f32p = ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p
        dp = ctypes.POINTER(AttnDesc)
        L.gpu_flash_attn_layer.argtypes = [vp] * 4 + [i] * 6 + [vp]
        L.gpu_flash_attn_opt_prefill_layer.argtypes = [vp] * 4 + [i] * 6 + [vp]
        L.gpu_flash_attn_gqa_layer.argtypes = [vp] * 4 + [i] * 7 + [vp]
        L.gpu_rope_layer.argtypes = [vp] * 5 + [i] * 6 + [vp]
        L.gpu_rope_single_layer.argtypes = [vp] * 3 + [i] * 6 + [vp]
        L.gpu_rope_kv_append_layer.argtypes = [dp] + [vp] * 7 + [i32p, i, i, vp]
        L.gpu_qkv_rope_kv_append_layer.argtypes = [dp] + [vp] * 4 + [ctypes.c_int64] * 2 + [vp, vp, i32p, i, i, vp]
        L.gpu_split_qkv_layer.argtypes = [vp] * 4 + [i] * 5 + [vp]
        L.gpu_bias_add_layer.argtypes = [vp] * 3 + [i, i, ctypes.c_int64, i, vp]
        L.gpu_attn_prefill_layer.argtypes = [dp] + [vp] * 4 + [i, i, vp]
        pp = ctypes.POINTER(KvPages)
        L.gpu_rope_kv_append_paged_layer.argtypes = [dp, pp] + [vp] * 7 + [i32p, i, i, vp]
        L.gpu_attn_prefill_paged_layer.argtypes = [dp, pp] + [vp] * 4 + [i, i, vp]
        L.gpu_attn_decode_paged_layer.argtypes = [dp, pp] + [vp] * 7 + [i32p, i, i, vp, ctypes.c_size_t, vp]
        L.gpu_attn_decode_layer.argtypes = [dp, vp, f32p, f32p] + [vp] * 6 + [i32p, i32p, i, i, vp,
                                                                               ctypes.c_size_t, vp]
        L.gpu_attn_decode_layer_noalloc.argtypes = [dp] + [vp] * 7 + [i32p, i32p, i, i, vp]
        L.gpu_attn_decode_plan_bytes.argtypes = [dp, i]
        L.gpu_attn_decode_plan_bytes.restype = ctypes.c_size_t
        L.gpu_attn_decode_plan.argtypes = [dp, i32p, i, i, vp, ctypes.c_size_t]
        L.gpu_attn_decode_plan_size.argtypes = [vp]
        L.gpu_attn_decode_plan_size.restype = ctypes.c_size_t
        L.gpu_attn_decode_plan_workspace_bytes.argtypes = [vp]
        L.gpu_attn_decode_plan_workspace_bytes.restype = ctypes.c_size_t
        L.gpu_attn_decode_planned_layer.argtypes = [dp, pp, vp, vp, vp, f32p, f32p] + [vp] * 6 + [i32p, vp,
                                                                                                 ctypes.c_size_t, vp]
        L.gpu_attn_decode_workspace_bytes.argtypes = [dp, i]
        L.gpu_attn_decode_workspace_bytes.restype = ctypes.c_size_t
        L.gpu_attn_merge_lse_layer.argtypes = [vp, f32p, f32p, i, i, i, i, vp]
        L.gpu_attn_merge_packed_layer.argtypes = [vp, f32p, i, i, i, i, vp]
        L.gpu_attn_xchg_buffer_bytes.argtypes = [i, i]
        L.gpu_attn_xchg_buffer_bytes.restype = ctypes.c_size_t
        L.gpu_attn_xchg_local_slot.argtypes = [vp, i, i, ctypes.c_uint32, i]
        L.gpu_attn_xchg_local_slot.restype = vp
        L.gpu_attn_xchg_merge_layer.argtypes = [vp, vp, ctypes.POINTER(vp), i, i, ctypes.c_uint32, i, i, i, vp]
        L.gpu_attn_decode_xchg_layer.argtypes = [dp] + [vp] * 7 + [i32p, i32p, i, i, vp, ctypes.c_size_t, vp,
                                                 ctypes.POINTER(vp), i, i, ctypes.c_uint32, vp]
        L.gpu_peer_buffer_alloc.argtypes = [ctypes.c_size_t, ctypes.POINTER(vp), ctypes.c_char_p]
        L.gpu_peer_buffer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp)]
        L.gpu_peer_buffer_close.argtypes = [vp]
        L.gpu_peer_buffer_free.argtypes = [vp]
        L.gpu_ops_set_workspace.argtypes = [vp, ctypes.c_size_t]
        L.gpu_attn_set_decode_chunk.argtypes = [i]
        L.gpu_attn_set_decode_early_prefetch.argtypes = [i]
        L.gpu_attn_set_prefill_kernel.argtypes = [i]
        L.gpu_attn_set_prefill_l2_window.argtypes = [ctypes.c_size_t]
        L.gpu_ops_launch_count.argtypes = [i]
        L.gpu_ops_launch_count.restype = ctypes.c_long
        L.gpu_ops_last_error_string.restype = ctypes.c_char_p
        _lib = L
    return _lib


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream):
    if stream is not None:
        return stream if isinstance(stream, int) else stream.cuda_stream
    import torch
    return torch.cuda.current_stream().cuda_stream


def _check(rc):
    if rc != 0:
        raise GpuOpsError("gpu_ops status %d: %s" % (rc, lib().gpu_ops_last_error_string().decode()))


def last_error_string():
    return lib().gpu_ops_last_error_string().decode()


def gpu_flash_attn_layer(output, q, k, v, m, n, offset, head_num, head_dim, dt, stream=None):
    _check(lib().gpu_flash_attn_layer(_ptr(output), _ptr(q), _ptr(k), _ptr(v), m, n, offset, head_num,
                                      head_dim, dt, _stream(stream)))


def gpu_flash_attn_opt_prefill_layer(output, q, k, v, m, n, offset, head_num, head_dim, dt, stream=None):
    _check(lib().gpu_flash_attn_opt_prefill_layer(_ptr(output), _ptr(q), _ptr(k), _ptr(v), m, n, offset,
                                                  head_num, head_dim, dt, _stream(stream)))


def gpu_flash_attn_gqa_layer(output, q, k, v, m, n, offset, group_size, kv_head_num, head_dim, dt,
                             stream=None):
    _check(lib().gpu_flash_attn_gqa_layer(_ptr(output), _ptr(q), _ptr(k), _ptr(v), m, n, offset, group_size,
                                          kv_head_num, head_dim, dt, _stream(stream)))


def gpu_rope_layer(output_q, output_k, freqs_cis, input_q, input_k, start_pos, cur_size, n_heads,
                   hidden_dim, is_neox_style, dt, stream=None):
    _check(lib().gpu_rope_layer(_ptr(output_q), _ptr(output_k), _ptr(freqs_cis), _ptr(input_q),
                                _ptr(input_k), start_pos, cur_size, n_heads, hidden_dim,
                                int(bool(is_neox_style)), dt, _stream(stream)))


def gpu_rope_single_layer(output_x, freqs_cis, input_x, start_pos, cur_size, n_heads, hidden_dim,
                          is_neox_style, dt, stream=None):
    _check(lib().gpu_rope_single_layer(_ptr(output_x), _ptr(freqs_cis), _ptr(input_x), start_pos, cur_size,
                                       n_heads, hidden_dim, int(bool(is_neox_style)), dt, _stream(stream)))


def gpu_rope_kv_append_layer(desc, q_out, k_cache, v_cache, q_in, k_in, v_in, freqs_cis, start_pos_dev,
                             start_pos, m, stream=None):
    _check(lib().gpu_rope_kv_append_layer(ctypes.byref(desc), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                          _ptr(q_in), _ptr(k_in), _ptr(v_in), _ptr(freqs_cis),
                                          _ptr(start_pos_dev), start_pos, m, _stream(stream)))


def gpu_qkv_rope_kv_append_layer(desc, q_out, k_cache, v_cache, qkv_in, qkv_seq_stride, qkv_tok_stride, qkv_bias,
                                 freqs_cis, start_pos_dev, start_pos, m, stream=None):
    """RoPE + append fed from a fused [q | k | v] projection row, optional bias row."""
    _check(lib().gpu_qkv_rope_kv_append_layer(ctypes.byref(desc), _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                              _ptr(qkv_in), qkv_seq_stride, qkv_tok_stride, _ptr(qkv_bias),
                                              _ptr(freqs_cis), _ptr(start_pos_dev), start_pos, m, _stream(stream)))


def gpu_bias_add_layer(out, x, bias, rows, width, row_stride, dt, stream=None):
    _check(lib().gpu_bias_add_layer(_ptr(out), _ptr(x), _ptr(bias), rows, width, row_stride, dt, _stream(stream)))


def gpu_split_qkv_layer(out_q, out_k, out_v, qkv, batch, q_dim, k_dim, v_dim, dt, stream=None):
    _check(lib().gpu_split_qkv_layer(_ptr(out_q), _ptr(out_k), _ptr(out_v), _ptr(qkv), batch, q_dim, k_dim, v_dim,
                                     dt, _stream(stream)))


def gpu_rope_kv_append_paged_layer(desc, pages, q_out, k_pool, v_pool, q_in, k_in, v_in, freqs_cis, start_pos_dev,
                                   start_pos, m, stream=None):
    _check(lib().gpu_rope_kv_append_paged_layer(ctypes.byref(desc), ctypes.byref(pages), _ptr(q_out), _ptr(k_pool),
                                                _ptr(v_pool), _ptr(q_in), _ptr(k_in), _ptr(v_in), _ptr(freqs_cis),
                                                _ptr(start_pos_dev), start_pos, m, _stream(stream)))


def gpu_attn_prefill_paged_layer(desc, pages, out, q, k_pool, v_pool, m, offset, stream=None):
    _check(lib().gpu_attn_prefill_paged_layer(ctypes.byref(desc), ctypes.byref(pages), _ptr(out), _ptr(q), _ptr(k_pool),
                                              _ptr(v_pool), m, offset, _stream(stream)))


def gpu_attn_decode_paged_layer(desc, pages, out, q_in, k_in, v_in, k_pool, v_pool, freqs_cis, kv_len_dev, append_new,
                                max_kv_len, workspace, workspace_bytes, stream=None):
    _check(lib().gpu_attn_decode_paged_layer(ctypes.byref(desc), ctypes.byref(pages), _ptr(out), _ptr(q_in),
                                             _ptr(k_in), _ptr(v_in), _ptr(k_pool), _ptr(v_pool), _ptr(freqs_cis),
                                             _ptr(kv_len_dev), int(bool(append_new)), max_kv_len, _ptr(workspace),
                                             workspace_bytes, _stream(stream)))


def gpu_attn_prefill_layer(desc, out, q, k_cache, v_cache, m, offset, stream=None):
    _check(lib().gpu_attn_prefill_layer(ctypes.byref(desc), _ptr(out), _ptr(q), _ptr(k_cache),
                                        _ptr(v_cache), m, offset, _stream(stream)))


def gpu_attn_decode_workspace_bytes(desc, max_kv_len):
    return int(lib().gpu_attn_decode_workspace_bytes(ctypes.byref(desc), max_kv_len))


def gpu_attn_decode_layer(desc, out, o_partial, lse_partial, q_in, k_in, v_in, k_cache, v_cache, freqs_cis,
                          kv_len_dev, rope_pos_dev, append_new, max_kv_len, workspace, workspace_bytes,
                          stream=None):
    _check(lib().gpu_attn_decode_layer(ctypes.byref(desc), _ptr(out), _ptr(o_partial), _ptr(lse_partial),
                                       _ptr(q_in), _ptr(k_in), _ptr(v_in), _ptr(k_cache), _ptr(v_cache),
                                       _ptr(freqs_cis), _ptr(kv_len_dev), _ptr(rope_pos_dev),
                                       int(bool(append_new)), max_kv_len, _ptr(workspace), workspace_bytes,
                                       _stream(stream)))


class DecodePlan:
    """Work partition of one decode step (gpu_attn_decode_plan): built from the
    host's cache lengths, the same for every layer of the step.  `host` is the
    blob as a numpy uint8 array; upload() copies it into a CUDA tensor."""

    def __init__(self, desc, kv_len_host, append_new, n_ctas=0):
        import numpy as np
        cap = int(lib().gpu_attn_decode_plan_bytes(ctypes.byref(desc), n_ctas))
        if cap == 0:
            raise GpuOpsError("gpu_attn_decode_plan_bytes: invalid arguments")
        lens = np.ascontiguousarray(np.asarray(kv_len_host, dtype=np.int32))
        buf = np.zeros(cap, dtype=np.uint8)
        _check(lib().gpu_attn_decode_plan(ctypes.byref(desc), lens.ctypes.data, int(bool(append_new)), n_ctas,
                                          buf.ctypes.data, cap))
        self.size = int(lib().gpu_attn_decode_plan_size(buf.ctypes.data))
        self.host = buf[:self.size].copy()
        self.workspace_bytes = int(lib().gpu_attn_decode_plan_workspace_bytes(self.host.ctypes.data))
        self.dev = None

    @property
    def header(self):
        """The plan header as a dict of its 32-bit fields."""
        import numpy as np
        w = self.host[:64].view(np.int32)
        names = ["magic", "n_ctas", "n_items", "n_groups", "n_slots", "batch", "n_kv_heads", "group", "append",
                 "max_total", "off_cta_begin", "off_items", "off_groups", "total_bytes", "total_tiles", "max_parts"]
        return dict(zip(names, (int(x) for x in w)))

    def tables(self):
        """(cta_begin, items [n][8], groups [n][4]) as numpy int32 arrays (for tests)."""
        import numpy as np
        h = self.header
        words = self.host.view(np.int32)
        cb = words[h["off_cta_begin"] // 4: h["off_cta_begin"] // 4 + h["n_ctas"] + 1]
        it = words[h["off_items"] // 4: h["off_items"] // 4 + 8 * h["n_items"]].reshape(-1, 8)
        mg = words[h["off_groups"] // 4: h["off_groups"] // 4 + 4 * h["n_groups"]].reshape(-1, 4)
        return cb, it, mg

    def upload(self, device=None):
        import torch
        self.dev = torch.from_numpy(self.host).to(device if device is not None else "cuda")
        return self.dev


def gpu_attn_decode_planned_layer(desc, pages, plan, out, o_partial, lse_partial, q_in, k_in, v_in, k_cache, v_cache,
                                  freqs_cis, rope_pos_dev, workspace, workspace_bytes, stream=None):
    """One fused decode step driven by a DecodePlan (upload() it first)."""
    _check(lib().gpu_attn_decode_planned_layer(ctypes.byref(desc), ctypes.byref(pages) if pages is not None else None,
                                               plan.host.ctypes.data, _ptr(plan.dev), _ptr(out), _ptr(o_partial),
                                               _ptr(lse_partial), _ptr(q_in), _ptr(k_in), _ptr(v_in), _ptr(k_cache),
                                               _ptr(v_cache), _ptr(freqs_cis), _ptr(rope_pos_dev), _ptr(workspace),
                                               workspace_bytes, _stream(stream)))


def gpu_attn_decode_noalloc_prepare():
    """Resolves the built-in scratch on the current device (takes its 16 MiB): call at start-up."""
    _check(lib().gpu_attn_decode_noalloc_prepare())


def gpu_attn_decode_layer_noalloc(desc, out, q_in, k_in, v_in, k_cache, v_cache, freqs_cis, kv_len_dev,
                                  rope_pos_dev, append_new, max_kv_len, stream=None):
    """The fused decode step with the library's built-in 16 MiB scratch: for callers
    that cannot allocate device memory.  Resolve the scratch at start-up
    (gpu_attn_decode_noalloc_prepare) before the host reserves the device memory and
    outside any stream capture; do not overlap calls on one device."""
    _check(lib().gpu_attn_decode_layer_noalloc(ctypes.byref(desc), _ptr(out), _ptr(q_in), _ptr(k_in),
                                               _ptr(v_in), _ptr(k_cache), _ptr(v_cache), _ptr(freqs_cis),
                                               _ptr(kv_len_dev), _ptr(rope_pos_dev), int(bool(append_new)),
                                               max_kv_len, _stream(stream)))


def gpu_peer_buffer_alloc(nbytes):
    """-> (device address, 64-byte handle to hand to the other processes of the node)."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    _check(lib().gpu_peer_buffer_alloc(nbytes, ctypes.byref(ptr), handle))
    return ptr.value, handle.raw


def gpu_peer_buffer_open(handle):
    ptr = ctypes.c_void_p()
    _check(lib().gpu_peer_buffer_open(handle, ctypes.byref(ptr)))
    return ptr.value


def gpu_peer_buffer_close(ptr):
    _check(lib().gpu_peer_buffer_close(ptr))


def gpu_peer_buffer_free(ptr):
    _check(lib().gpu_peer_buffer_free(ptr))


def gpu_attn_xchg_buffer_bytes(world, rows):
    return int(lib().gpu_attn_xchg_buffer_bytes(world, rows))


def gpu_attn_xchg_local_slot(local_buffer, world, rank, epoch, rows):
    return lib().gpu_attn_xchg_local_slot(local_buffer, world, rank, epoch, rows)


def gpu_attn_xchg_merge_layer(out, local_buffer, peer_buffers, world, rank, epoch, rows, head_dim, dt, stream=None):
    arr = (ctypes.c_void_p * world)(*[p for p in peer_buffers])
    _check(lib().gpu_attn_xchg_merge_layer(_ptr(out), local_buffer, arr, world, rank, epoch, rows, head_dim, dt,
                                           _stream(stream)))


def gpu_attn_decode_xchg_layer(desc, out, q_in, k_in, v_in, k_cache, v_cache, freqs_cis, kv_len_dev, rope_pos_dev,
                               append_new, max_kv_len, workspace, workspace_bytes, local_buffer, peer_buffers, world,
                               rank, epoch, stream=None):
    arr = (ctypes.c_void_p * world)(*[p for p in peer_buffers])
    _check(lib().gpu_attn_decode_xchg_layer(ctypes.byref(desc), _ptr(out), _ptr(q_in), _ptr(k_in), _ptr(v_in),
                                            _ptr(k_cache), _ptr(v_cache), _ptr(freqs_cis), _ptr(kv_len_dev),
                                            _ptr(rope_pos_dev), int(bool(append_new)), max_kv_len, _ptr(workspace),
                                            workspace_bytes, local_buffer, arr, world, rank, epoch, _stream(stream)))


def gpu_attn_merge_lse_layer(out, o_parts, lse_parts, n_parts, rows, head_dim, dt, stream=None):
    _check(lib().gpu_attn_merge_lse_layer(_ptr(out), _ptr(o_parts), _ptr(lse_parts), n_parts, rows,
                                          head_dim, dt, _stream(stream)))


def gpu_attn_merge_packed_layer(out, parts, n_parts, rows, head_dim, dt, stream=None):
    _check(lib().gpu_attn_merge_packed_layer(_ptr(out), _ptr(parts), n_parts, rows, head_dim, dt, _stream(stream)))


def gpu_ops_set_workspace(workspace, nbytes):
    _check(lib().gpu_ops_set_workspace(_ptr(workspace), nbytes))


def gpu_attn_set_decode_early_prefetch(on):
    _check(lib().gpu_attn_set_decode_early_prefetch(int(bool(on))))


def gpu_attn_set_decode_chunk(positions):
    _check(lib().gpu_attn_set_decode_chunk(positions))


def gpu_attn_set_prefill_kernel(which):
    _check(lib().gpu_attn_set_prefill_kernel(which))


def gpu_attn_set_prefill_l2_window(nbytes):
    """K/V bytes a chunk of (sequence, head) pairs may share in L2 (CTA order of the tcgen05 prefill kernel); 0 = default."""
    _check(lib().gpu_attn_set_prefill_l2_window(nbytes))


def gpu_attn_last_prefill_kernel():
    return int(lib().gpu_attn_last_prefill_kernel())


def gpu_ops_clear_kernel_status():
    _check(lib().gpu_ops_clear_kernel_status())


def gpu_ops_kernel_status():
    return int(lib().gpu_ops_kernel_status())


def gpu_ops_launch_count(reset=False):
    return int(lib().gpu_ops_launch_count(int(bool(reset))))
