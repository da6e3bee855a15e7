// Device helpers shared by the attention kernels: 16-bit type traits, the
// shared-memory swizzle, cp.async, ldmatrix and the warp-level mma.sync tile.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200attn {

constexpr int kHeadDim = 128;               // elements per head
constexpr int kRowBytes = kHeadDim * 2;     // one K/V/Q row in shared memory
constexpr float kLog2e = 1.4426950408889634f;

// ---------------------------------------------------------------------------
// 16-bit element traits
// ---------------------------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<__half> {
  using T2 = __half2;
  static __device__ __forceinline__ float to_f32(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f32(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2 *>(&u));
  }
};
template <> struct Elem<__nv_bfloat16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
  }
};

// ---------------------------------------------------------------------------
// RoPE of one pair, with the reference tests' operation order
// (tests/rope_single_layer_test.cpp:93-94): two fp32 products, one subtraction
// / addition, no fused multiply-add, so the result is bit-identical to a CPU
// evaluation of the same expressions.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void rope_pair(float a, float b, float c, float s, float &oa, float &ob) {
  oa = __fsub_rn(__fmul_rn(a, c), __fmul_rn(b, s));
  ob = __fadd_rn(__fmul_rn(a, s), __fmul_rn(b, c));
}

// Rotate the eight pairs f = 8i .. 8i+7 of one 128-element head row.  u0 / u1
// are the two 16-byte chunks that hold them: chunks (2i, 2i+1) for the
// interleaved pairing (2f, 2f+1), chunks (i, i+8) for the neox pairing
// (f, f+64).  tab points at the (cos, sin) entries of pair 8i.
template <typename T>
__device__ __forceinline__ void rope_chunk_pair(uint4 &u0, uint4 &u1, const float4 *tab, bool neox) {
  uint32_t *w0 = reinterpret_cast<uint32_t *>(&u0);
  uint32_t *w1 = reinterpret_cast<uint32_t *>(&u1);
  if (neox) {
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const float4 cs = tab[e2]; // (cos, sin) of pairs 2*e2 and 2*e2+1
      const float2 a = Elem<T>::unpack(w0[e2]);
      const float2 b = Elem<T>::unpack(w1[e2]);
      float oa0, ob0, oa1, ob1;
      rope_pair(a.x, b.x, cs.x, cs.y, oa0, ob0);
      rope_pair(a.y, b.y, cs.z, cs.w, oa1, ob1);
      w0[e2] = Elem<T>::pack(oa0, oa1);
      w1[e2] = Elem<T>::pack(ob0, ob1);
    }
  } else {
#pragma unroll
    for (int e2 = 0; e2 < 4; ++e2) {
      const float4 cs = tab[e2];
      uint32_t *w = (e2 < 2) ? (w0 + 2 * e2) : (w1 + 2 * (e2 - 2));
      const float2 x0 = Elem<T>::unpack(w[0]);
      const float2 x1 = Elem<T>::unpack(w[1]);
      float oa0, ob0, oa1, ob1;
      rope_pair(x0.x, x0.y, cs.x, cs.y, oa0, ob0);
      rope_pair(x1.x, x1.y, cs.z, cs.w, oa1, ob1);
      w[0] = Elem<T>::pack(oa0, ob0);
      w[1] = Elem<T>::pack(oa1, ob1);
    }
  }
}

// ---------------------------------------------------------------------------
// Shared-memory layout of a [rows][128] 16-bit tile: 256-byte rows of sixteen
// 16-byte chunks; chunk c of row r is stored at chunk position c ^ (r & 7), so
// that the eight rows an ldmatrix touches fall into eight different bank groups.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
  return static_cast<uint32_t>(row * kRowBytes + ((chunk ^ (row & 7)) << 4));
}

// Layout of a K/V tile written by TMA with the 128-byte swizzle: two half tiles of
// [rows][64 elements] (128-byte rows), the second HALF_BYTES after the first; the 16-byte chunk
// c of a 128-byte row sits at chunk position c ^ (row & 7).  HALF_BYTES == 0 selects the
// 256-byte-row layout above.
template <int HALF_BYTES> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  if (HALF_BYTES == 0) return swz_off(row, chunk);
  return static_cast<uint32_t>((chunk >> 3) * HALF_BYTES + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous copy global -> shared; src_bytes = 0 zero-fills.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D (16x8, fp32) += A (16x16) * B (16x8), 16-bit operands.
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------
// One warp's online-softmax state for 16 query rows: thread `lane` owns rows
// lane/4 (index 0) and lane/4 + 8 (index 1); o[nt][0..1] are row 0's columns
// nt*8 + 2*(lane%4) + {0,1}, o[nt][2..3] the same columns of row 1.
// Scores are kept in the log2 domain (score * scale * log2(e)).
// ---------------------------------------------------------------------------
struct WarpAcc {
  float o[16][4];
  float mx[2];
  float sum[2]; // this thread's partial row sums (reduced over the quad at the end)
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    mx[0] = mx[1] = -INFINITY;
    sum[0] = sum[1] = 0.f;
  }
};

// Load the A fragments (16 rows x 128) of a swizzled Q tile whose first row is
// `row0` into registers: qa[ks] covers d = 16*ks .. 16*ks+15.
__device__ __forceinline__ void load_q_frags(uint32_t (&qa)[8][4], uint32_t q_smem, int row0, int lane) {
  const int j = lane >> 3, r = lane & 7;
  const int row = row0 + (j & 1) * 8 + r;
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    ldmatrix_x4(qa[ks], q_smem + swz_off(row, 2 * ks + (j >> 1)));
  }
}

// One warp: S = Q (16 x 128) . K^T for NT*8 key positions starting at tile row
// `krow0` of a swizzled K tile, mask, online softmax, O += P . V.
//   col0:      global position of tile row krow0
//   col_end:   positions >= col_end are masked for every row
//   lim0/lim1: per-row causal limits (positions >= lim are masked) of the
//              thread's two rows
//   scale_log2: softmax scale * log2(e)
//   HALF_BYTES: layout of the K / V tiles (see tile_off)
template <typename T, int NT, int HALF_BYTES = 0>
__device__ __forceinline__ void warp_tile(WarpAcc &acc, const uint32_t (&qa)[8][4], uint32_t k_smem,
                                          uint32_t v_smem, int krow0, int col0, int col_end, int lim0,
                                          int lim1, float scale_log2, int lane) {
  static_assert(NT % 2 == 0, "key positions are consumed 16 at a time");
  float s[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;

  const int j = lane >> 3, r = lane & 7;
  // ---- S = Q K^T ----
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t kb[4];
      const int row = krow0 + np * 16 + (j >> 1) * 8 + r;
      ldmatrix_x4(kb, k_smem + tile_off<HALF_BYTES>(row, 2 * ks + (j & 1)));
      mma_16816<T>(s[2 * np], qa[ks], kb[0], kb[1]);
      mma_16816<T>(s[2 * np + 1], qa[ks], kb[2], kb[3]);
    }
  }
  // ---- mask + running max ----
  const int cbase = col0 + 2 * (lane & 3);
  const int e0 = min(lim0, col_end), e1 = min(lim1, col_end);
  float tmax0 = -INFINITY, tmax1 = -INFINITY;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int c = cbase + nt * 8;
    s[nt][0] = (c < e0) ? s[nt][0] * scale_log2 : -INFINITY;
    s[nt][1] = (c + 1 < e0) ? s[nt][1] * scale_log2 : -INFINITY;
    s[nt][2] = (c < e1) ? s[nt][2] * scale_log2 : -INFINITY;
    s[nt][3] = (c + 1 < e1) ? s[nt][3] * scale_log2 : -INFINITY;
    tmax0 = fmaxf(tmax0, fmaxf(s[nt][0], s[nt][1]));
    tmax1 = fmaxf(tmax1, fmaxf(s[nt][2], s[nt][3]));
  }
  tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 1));
  tmax0 = fmaxf(tmax0, __shfl_xor_sync(0xffffffffu, tmax0, 2));
  tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 1));
  tmax1 = fmaxf(tmax1, __shfl_xor_sync(0xffffffffu, tmax1, 2));
  const float mnew0 = fmaxf(acc.mx[0], tmax0), mnew1 = fmaxf(acc.mx[1], tmax1);
  // a row with nothing visible so far keeps max = -inf; subtract 0 instead so exp2 gives 0, not NaN
  const float msub0 = (mnew0 == -INFINITY) ? 0.f : mnew0;
  const float msub1 = (mnew1 == -INFINITY) ? 0.f : mnew1;
  const float corr0 = exp2f(acc.mx[0] - msub0), corr1 = exp2f(acc.mx[1] - msub1);
  acc.mx[0] = mnew0;
  acc.mx[1] = mnew1;
  acc.sum[0] *= corr0;
  acc.sum[1] *= corr1;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    acc.o[i][0] *= corr0;
    acc.o[i][1] *= corr0;
    acc.o[i][2] *= corr1;
    acc.o[i][3] *= corr1;
  }
  // ---- P = exp2(S - max), packed as A fragments ----
  uint32_t pa[NT / 2][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const float p0 = exp2f(s[nt][0] - msub0), p1 = exp2f(s[nt][1] - msub0);
    const float p2 = exp2f(s[nt][2] - msub1), p3 = exp2f(s[nt][3] - msub1);
    acc.sum[0] += p0 + p1;
    acc.sum[1] += p2 + p3;
    pa[nt >> 1][(nt & 1) * 2 + 0] = Elem<T>::pack(p0, p1);
    pa[nt >> 1][(nt & 1) * 2 + 1] = Elem<T>::pack(p2, p3);
  }
  // ---- O += P V ----
#pragma unroll
  for (int kp = 0; kp < NT / 2; ++kp) {
    const int row = krow0 + kp * 16 + (j & 1) * 8 + r;
#pragma unroll
    for (int dp = 0; dp < 8; ++dp) {
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, v_smem + tile_off<HALF_BYTES>(row, 2 * dp + (j >> 1)));
      mma_16816<T>(acc.o[2 * dp], pa[kp], vb[0], vb[1]);
      mma_16816<T>(acc.o[2 * dp + 1], pa[kp], vb[2], vb[3]);
    }
  }
}

} // namespace b200attn
