// Building blocks of the bf16 attention kernels that run on mma.sync.m16n8k16 (bf16 in, fp32
// accumulate), compiled for one head size (-DGF_HEAD_DIM=<multiple of 16, at most 256>): K/V tiles
// of 64 keys gathered from the paged cache by cp.async, Q*K^T and P*V tile products read by
// ldmatrix, and the online-softmax update.  Used by a group of 128 threads (four warps); `tid` is
// the thread's index inside that group.
#pragma once
#include "common.cuh"

#ifndef GF_HEAD_DIM
#define GF_HEAD_DIM 128
#endif

namespace gf {

constexpr int HD = GF_HEAD_DIM;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16, <= 256");
constexpr int ROW = HD + 8;          // padded smem row (elements): 16-byte chunks, odd chunk stride
constexpr int KT = 64;               // keys per tile
constexpr int NTHREADS = 128;
constexpr int KCH = HD / 16;         // 16-wide chunks of the head size
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool pred) {
  const int n = pred ? 16 : 0;       // src-size 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src),
               "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Load keys [c0, c0 + KT) of one kv head into [KT][ROW] tiles of K and V; rows at or past `end` (or
// before `begin`) are zero-filled and touch no page.  `tbl[lp - lp_base]` is the physical page of
// logical page lp: the kernels copy the part of the request's block table they need into shared
// memory first (lp_base = its first entry), so a tile's loads do not wait for look-ups in global
// memory; the look-ups of all of a thread's rows are issued before its copies.
__device__ __forceinline__ void load_kv_tiles(bf16* kdst, bf16* vdst,
                                              const bf16* __restrict__ kpages,
                                              const bf16* __restrict__ vpages,
                                              const int* tbl, int lp_base, int c0,
                                              int begin, int end, int page_size, int page_shift,
                                              size_t tok_stride, int kvh, int tid) {
  constexpr int CH = HD / 8;                           // 16-byte chunks in a row
  if constexpr (NTHREADS % CH == 0) {
    // a thread keeps its chunk column and walks down the rows in steps of NTHREADS / CH
    constexpr int RSTEP = NTHREADS / CH, ITERS = KT / RSTEP;
    const int ch = tid % CH, rb = tid / CH;
    const unsigned col = (unsigned)(kvh * HD + ch * 8);
    const unsigned stride = (unsigned)tok_stride;
    unsigned slot[ITERS];
    bool ok[ITERS];
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int c = c0 + rb + it * RSTEP;
      ok[it] = c >= begin && c < end;
      slot[it] = 0;
      if (ok[it]) {
        const int lp = page_shift >= 0 ? c >> page_shift : c / page_size;
        const int in_page = page_shift >= 0 ? c & (page_size - 1) : c - lp * page_size;
        slot[it] = (unsigned)tbl[lp - lp_base] * (unsigned)page_size + (unsigned)in_page;
      }
    }
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const size_t off = (size_t)slot[it] * stride + col;        // one wide multiply
      const int r = rb + it * RSTEP;
      cp_async16(kdst + r * ROW + ch * 8, kpages + off, ok[it]);
      cp_async16(vdst + r * ROW + ch * 8, vpages + off, ok[it]);
    }
  } else {
    constexpr int ITERS = (KT * CH + NTHREADS - 1) / NTHREADS;
#pragma unroll
    for (int it = 0; it < ITERS; ++it) {
      const int i = tid + it * NTHREADS;
      if (i >= KT * CH) break;
      const int r = i / CH, ch = i - r * CH;
      const int c = c0 + r;
      const bool ok = c >= begin && c < end;
      size_t off = 0;
      if (ok) {
        const int lp = c / page_size;
        off = ((size_t)tbl[lp - lp_base] * page_size + (c - lp * page_size)) * tok_stride +
              (size_t)(kvh * HD + ch * 8);
      }
      cp_async16(kdst + r * ROW + ch * 8, kpages + off, ok);
      cp_async16(vdst + r * ROW + ch * 8, vpages + off, ok);
    }
  }
}

// S[16 x (8*NT)] += A(16 x HD) * K^T for the keys of rows [key0, key0 + 8*NT) of the tile.
template <int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const uint32_t (&qf)[KCH][4],
                                        const bf16* ktile, int key0, int lane) {
  static_assert(NT % 2 == 0, "");
  const int mi = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kc = 0; kc < KCH; ++kc) {
#pragma unroll
    for (int n2 = 0; n2 < NT / 2; ++n2) {
      uint32_t b[4];
      ldsm_x4(b, ktile + (key0 + n2 * 16 + (mi >> 1) * 8 + r) * ROW + kc * 16 + (mi & 1) * 8);
      mma16816(s[2 * n2], qf[kc], b[0], b[1]);
      mma16816(s[2 * n2 + 1], qf[kc], b[2], b[3]);
    }
  }
}

// O[16 x HD] += P(16 x 8*NT, bf16 from s) * V for the keys of rows [key0, key0 + 8*NT) of the tile.
template <int NT>
__device__ __forceinline__ void pv_tile(float (&o)[HD / 8][4], const float (&s)[NT][4],
                                        const bf16* vtile, int key0, int lane) {
  const int mi = lane >> 3, r = lane & 7;
#pragma unroll
  for (int kc = 0; kc < NT / 2; ++kc) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kc][0], s[2 * kc][1]);
    a[1] = pack_bf16(s[2 * kc][2], s[2 * kc][3]);
    a[2] = pack_bf16(s[2 * kc + 1][0], s[2 * kc + 1][1]);
    a[3] = pack_bf16(s[2 * kc + 1][2], s[2 * kc + 1][3]);
#pragma unroll
    for (int n2 = 0; n2 < HD / 16; ++n2) {
      uint32_t b[4];
      ldsm_x4_t(b, vtile + (key0 + kc * 16 + (mi & 1) * 8 + r) * ROW + n2 * 16 + (mi >> 1) * 8);
      mma16816(o[2 * n2], a, b[0], b[1]);
      mma16816(o[2 * n2 + 1], a, b[2], b[3]);
    }
  }
}

// One online-softmax update of a warp's 16 rows over 8*NT keys.  s holds raw dot products on
// entry and the probabilities on exit.  Columns are keys col0 + ...; row i of the pair (i = 0:
// row g, i = 1: row g + 8) sees keys in [lo[i], hi[i]].  m and l are per-thread copies of the row
// maximum (in log2 units) and a partial row sum.
__device__ __forceinline__ float fast_exp2(float x) {   // 2^x; -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// MASKED = false: every column is visible to both rows (an interior tile): no comparisons.
template <int NT, bool MASKED>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&o)[HD / 8][4],
                                               float (&m)[2], float (&l)[2], int col0,
                                               const int (&lo)[2], const int (&hi)[2],
                                               float scale_log2, int lane) {
  const int t = lane & 3;
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      float v = s[j][e] * scale_log2;
      if (MASKED) {
        const int c = col0 + 8 * j + 2 * t + (e & 1);
        v = (c >= lo[i] && c <= hi[i]) ? v : -INFINITY;
      }
      s[j][e] = v;
      mx[i] = fmaxf(mx[i], v);
    }
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
  }
  float corr[2], mnew[2], msub[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    mnew[i] = fmaxf(m[i], mx[i]);
    msub[i] = mnew[i] == -INFINITY ? 0.f : mnew[i];      // keeps -inf - -inf out of the exponent
    corr[i] = fast_exp2(m[i] - msub[i]);                 // m = -inf: 0 (nothing accumulated yet)
    m[i] = mnew[i];
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = e >> 1;
      const float p = fast_exp2(s[j][e] - msub[i]);
      s[j][e] = p;
      sum[i] += p;
    }
#pragma unroll
  for (int i = 0; i < 2; ++i) l[i] = l[i] * corr[i] + sum[i];
  // the accumulator is rescaled only when some row of the warp got a new maximum
  if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
      o[n][0] *= corr[0];
      o[n][1] *= corr[0];
      o[n][2] *= corr[1];
      o[n][3] *= corr[1];
    }
  }
}

}  // namespace gf
