// All transformer layers of one decode step (at most 16 requests, one token each) in ONE
// persistent kernel, compiled for one head size (-DGF_HEAD_DIM=<multiple of 16, at most 256>).
//
// A layer here is: RMS norm -> joined q/k/v product (+ bias) -> rotary encoding, K/V written to
// their cache page, attention over the paged cache -> output product added to the residual ->
// RMS norm -> gate/up product with SiLU(gate) * up -> down product added to the residual; the
// reference runs the same sequence as about a dozen launches a layer
// (ginfer/core/layer/transformer/encoder.cc:33-39, attention.cc:45-82, feed_forward.cc).
//
// One CTA per SM, launched cooperatively.  Inside a CTA:
//   warp 0    streams the weight tiles this CTA will need, through a ring of 16 KB stages, by TMA.
//             Weights do not depend on anything computed in the step, so it runs ahead of the
//             phases as far as the ring allows and the memory system never waits for a phase.
//   warp 1    issues tcgen05.mma: weights are the A operand (128 rows = TMEM lanes), the tokens the
//             16 columns of the accumulator in tensor memory.
//   warps 2-9 build the activation operand of each product in shared memory (normalising the fp32
//             residual on the way where a norm precedes the product), drain the accumulator, and
//             run attention (mma.sync, csrc/attention_mma.cuh) between the products.
// The phases of a layer (q/k/v, attention, output, gate/up, down) are separated by barriers over
// the whole grid.  Work inside a phase is split into items (a tile of 128 weight rows, a range
// of the reduction dimension) dealt to CTAs round robin; partial sums of a split reduction go
// through a workspace and are added up in split order by whichever CTA finishes a tile last, so
// the result does not depend on timing.  The residual stream stays in fp32; what the unfused
// kernels round to bf16 (normalised activations, q/k/v, attention output, gate*up) is rounded here
// at the same places.
//
// Every wait (mbarrier, grid barrier) is bounded: when one runs out, the kernel records a code in
// `err`, every CTA sees it at its next barrier and leaves.
#include <cstring>

#include "attention_mma.cuh"
#include "tc_common.cuh"

namespace gf {

constexpr int DL_THREADS = 320;
constexpr int DL_WORKERS = 256;
constexpr int DL_BN = 16;                       // token columns of every product
constexpr int DL_MAX_TOKENS = 16;
constexpr uint32_t DL_A_BYTES = BM * BK * 2;    // one weight tile: 16 KB
constexpr uint32_t DL_B_BYTES = DL_BN * BK * 2; // one k block of the activation operand: 2 KB
constexpr int DL_ATT_STAGES = 2;
constexpr int DL_MAX_SPLITS = 16;               // of a product's reduction, and of a request's keys

enum { PH_QKV = 0, PH_ATT = 1, PH_OUT = 2, PH_GATEUP = 3, PH_DOWN = 4 };

struct alignas(64) DlLayer {
  CUtensorMap w[4];            // q/k/v, output, gate/up (rows interleaved), down: [N, K] bf16
  const float* bias[4];        // fp32 or null
  const void* gamma[2];        // norm before the mixer, norm before the feed-forward
  int gamma_f32[2];
  float eps[2];
  bf16* kpages;                // [pages][page][kv heads][head size]
  bf16* vpages;
  int group;                   // which of the step's block tables this cache goes by
  int window;                  // 0: every key is visible
  int write_cache;             // 0: the layer reads a cache that another layer writes
  int pad_;
};
constexpr int DL_MAX_GROUPS = 4;

struct DlPhase {
  int N, KB, per, S, off, items;   // rows, k blocks, k blocks per split, splits, first CTA, N tiles * S
};

struct DlParams {
  const DlLayer* layers;
  int num_layers, M, H, NH, NKV, I, NQKV, page_size, rot;
  float scale_log2;
  DlPhase ph[4];               // q/k/v, output, gate/up, down
  int attn_splits, attn_chunks, attn_items;
  int stages;                  // depth of the weight ring
  uint32_t u_bytes;            // shared memory that the operand and attention share
  int tbl_cap;                 // block-table entries an attention item copies to shared memory
  int stop_layer, stop_phase;  // leave after this phase of this layer (testing); -1: run everything
  const int* token_ids;        // [M]; with emb: the residual starts as the embedding rows
  const bf16* emb;             // [vocab, H] or null (then h is given)
  const int* positions;        // [M]
  const float* rope;           // [positions][rot]: cos | sin, or null
  const int* block_table[DL_MAX_GROUPS];   // [requests of the step][table_stride], per cache group
  int table_stride[DL_MAX_GROUPS];
  float* h;                    // [16, H] fp32 residual stream, in and out
  float* ws_qkv;               // [S][16][NQKV]
  bf16* qkv;                   // [16][NQKV]: the q/k/v product with its bias
  float* att_o;                // [M][NH][splits][HD]
  float* att_ml;               // [M][NH][splits][2]
  bf16* attn_out;              // [16][NH * HD]
  float* ws_red;               // [S][16][H]
  bf16* z;                     // [16][I]
  unsigned int* counters;      // tiles of the output / down products, attention groups
  unsigned int* bar;           // grid barrier: arrivals
  int* err;
  unsigned long long* stamps;  // [CTAs][64] nanosecond time stamps of the first phases, or null
};
__device__ __forceinline__ void dl_stamp(const DlParams& p, int idx) {
  if (p.stamps && idx < 64) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.stamps[(size_t)blockIdx.x * 64 + idx] = t;
  }
}

__device__ __forceinline__ void named_bar(int id, int n) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ unsigned int ld_acquire(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float bf16_round(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
// silu(gate) * up on the bf16-rounded products, as the separate activation kernel computes it
__device__ __forceinline__ float dl_silu_mul(float g, float u) {
  const float gg = bf16_round(g), uu = bf16_round(u);
  return gg * (1.0f / (1.0f + expf(-gg))) * uu;
}

struct DlItem {
  int layer, phase, n0, kb0, nkb, r, s;
};
// The weight-bearing items of this CTA in the order in which it meets them: layer by layer,
// phase by phase, round robin inside a phase.  The producer, the MMA issuer and the workers walk
// the same sequence.
struct DlItemIter {
  int layer = 0, phase = 0, idx = -1;
  __device__ bool next(const DlParams& p, int cta, int ncta, DlItem& it) {
    constexpr int overall[4] = {PH_QKV, PH_OUT, PH_GATEUP, PH_DOWN};
    for (;;) {
      if (layer >= p.num_layers) return false;
      if (p.stop_layer >= 0 &&
          (layer > p.stop_layer || (layer == p.stop_layer && overall[phase] > p.stop_phase)))
        return false;
      const DlPhase& ph = p.ph[phase];
      if (idx < 0) idx = (cta - ph.off % ncta + ncta) % ncta;
      if (idx < ph.items) {
        it.layer = layer, it.phase = phase;
        it.r = idx / ph.S, it.s = idx - it.r * ph.S;
        it.n0 = it.r * BM;
        it.kb0 = it.s * ph.per;
        it.nkb = min(ph.per, ph.KB - it.kb0);
        idx += ncta;
        return true;
      }
      idx = -1;
      if (++phase == 4) phase = 0, ++layer;
    }
  }
};

struct DlShared {
  unsigned char* ring;
  unsigned char* U;
  uint64_t* full;
  uint64_t* empty;
  uint64_t* b_ready;
  uint64_t* acc_full;
  uint32_t* tmem_slot;
  volatile int* dead;          // a wait ran out somewhere: leave
  volatile int* issued;        // weight stages the producer has asked for
  int* flag;                   // broadcast of "this CTA finished the tile last"
  float* rms;                  // [16]
};

// ----------------------------------------------------------------------------- grid barrier
// Arrivals are counted in one word that only grows: the n-th barrier is passed when it reaches
// n * CTAs.  Called by the 256 workers; the other two warps are paced by mbarriers.
__device__ __forceinline__ bool grid_barrier(const DlParams& p, DlShared& sh, unsigned int& epoch,
                                             int wt) {
  named_bar(1, DL_WORKERS);
  if (wt == 0) {
    __threadfence();
    atomicAdd(p.bar, 1u);
    const unsigned int target = (++epoch) * gridDim.x;
    bool ok = false;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
      if (ld_acquire(p.bar) >= target) {
        ok = true;
        break;
      }
      if ((spin & 63) == 63 && *reinterpret_cast<volatile int*>(p.err) != 0) break;
      if (spin > 256) __nanosleep(40);
    }
    if (!ok) {
      atomicCAS(p.err, 0, 20);
      *sh.dead = 1;
    }
    __threadfence();
  } else {
    ++epoch;
  }
  named_bar(1, DL_WORKERS);
  return *sh.dead == 0;
}

// ----------------------------------------------------------------------------- operands
// bres[kb][token][64] bf16 in the 128-byte-swizzled layout of a K-major tcgen05 operand.
__device__ __forceinline__ unsigned char* b_chunk(unsigned char* bres, int kbl, int m, int ch) {
  return bres + (size_t)kbl * DL_B_BYTES + m * 128 + ((ch ^ (m & 7)) << 4);
}

// rms of every token's row of the fp32 residual: 16 threads a token, a fixed shuffle tree.
__device__ __forceinline__ void row_rms(const DlParams& p, DlShared& sh, float eps, int wt) {
  const int m = wt >> 4, sub = wt & 15;
  float ss = 0.f;
  if (m < p.M) {
    const float* row = p.h + (size_t)m * p.H;
#pragma unroll 8
    for (int c = sub * 4; c < p.H; c += 64) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(row + c));
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (sub == 0) sh.rms[m] = sqrtf(ss / (float)p.H + eps);
  named_bar(1, DL_WORKERS);
}

// The k blocks [kb0, kb0 + nkb) of bf16(h * gamma / rms) for every token.
__device__ __forceinline__ void build_normed(const DlParams& p, DlShared& sh, const void* gamma,
                                             int gamma_f32, int kb0, int nkb, int wt) {
  const int ch = wt & 7, m = (wt >> 3) & 15, kb_first = wt >> 7;      // 2 k blocks a pass
  const bool live = m < p.M;
  const float r = live ? sh.rms[m] : 1.f;
  for (int kbl = kb_first; kbl < nkb; kbl += 8) {
    float4 s0[4], s1[4], g0[4], g1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = min((kb0 + min(kbl + 2 * u, nkb - 1)) * BK + ch * 8, p.H - 8);
      const float4* sp = reinterpret_cast<const float4*>(p.h + (size_t)(live ? m : 0) * p.H + k);
      s0[u] = __ldcg(sp);
      s1[u] = __ldcg(sp + 1);
      if (gamma_f32) {
        g0[u] = __ldg(reinterpret_cast<const float4*>((const float*)gamma + k));
        g1[u] = __ldg(reinterpret_cast<const float4*>((const float*)gamma + k + 4));
      } else {
        const uint4 gr = __ldg(reinterpret_cast<const uint4*>((const bf16*)gamma + k));
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
        const float2 a0 = __bfloat1622float2(gp[0]), a1 = __bfloat1622float2(gp[1]);
        const float2 a2 = __bfloat1622float2(gp[2]), a3 = __bfloat1622float2(gp[3]);
        g0[u] = make_float4(a0.x, a0.y, a1.x, a1.y);
        g1[u] = make_float4(a2.x, a2.y, a3.x, a3.y);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int kk = kbl + 2 * u;
      if (kk >= nkb) break;
      const int k = (kb0 + kk) * BK + ch * 8;
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      if (live && k < p.H) {
        w.x = pack_bf16(s0[u].x * g0[u].x / r, s0[u].y * g0[u].y / r);
        w.y = pack_bf16(s0[u].z * g0[u].z / r, s0[u].w * g0[u].w / r);
        w.z = pack_bf16(s1[u].x * g1[u].x / r, s1[u].y * g1[u].y / r);
        w.w = pack_bf16(s1[u].z * g1[u].z / r, s1[u].w * g1[u].w / r);
      }
      *reinterpret_cast<uint4*>(b_chunk(sh.U, kk, m, ch)) = w;
    }
  }
}

// The same in one pass for rows that fit in registers: TPT threads a token hold the token's whole
// fp32 row (and gamma), add up its squares with shuffles, and write the k blocks of the range.
// One round trip to memory instead of a pass for the statistics and one for the operand.
constexpr int DL_ROW_OCTETS = 12;      // 8-channel groups a thread holds at most
template <int TPT, int CAP>
__device__ __noinline__ void build_normed_once(const DlParams& p, DlShared& sh,
                                                  const void* gamma, int gamma_f32, float eps,
                                                  int kb0, int nkb, int wt) {
  const int m = wt / TPT, l = wt % TPT;
  const int noct = p.H >> 3;
  const bool live = m < p.M;
  const float* row = p.h + (size_t)(live ? m : 0) * p.H;
  float4 a[CAP][2];
  uint4 g[CAP];
#pragma unroll
  for (int i = 0; i < CAP; ++i) {
    const int o = min(l + TPT * i, noct - 1);
    a[i][0] = __ldcg(reinterpret_cast<const float4*>(row + o * 8));
    a[i][1] = __ldcg(reinterpret_cast<const float4*>(row + o * 8 + 4));
  }
  if (!gamma_f32) {
#pragma unroll
    for (int i = 0; i < CAP; ++i)
      g[i] = __ldg(reinterpret_cast<const uint4*>((const bf16*)gamma + min(l + TPT * i, noct - 1) * 8));
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < CAP; ++i)
    if (l + TPT * i < noct)
      ss += a[i][0].x * a[i][0].x + a[i][0].y * a[i][0].y + a[i][0].z * a[i][0].z +
            a[i][0].w * a[i][0].w + a[i][1].x * a[i][1].x + a[i][1].y * a[i][1].y +
            a[i][1].z * a[i][1].z + a[i][1].w * a[i][1].w;
#pragma unroll
  for (int o = TPT / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = sqrtf(ss / (float)p.H + eps);
#pragma unroll
  for (int i = 0; i < CAP; ++i) {
    const int o = l + TPT * i;                  // octets past the row's end are written as zeros
    const int kbl = (o >> 3) - kb0;
    if (kbl < 0 || kbl >= nkb) continue;
    uint4 w = make_uint4(0u, 0u, 0u, 0u);
    if (live && o < noct) {
      float4 g0, g1;
      if (gamma_f32) {
        g0 = __ldg(reinterpret_cast<const float4*>((const float*)gamma + o * 8));
        g1 = __ldg(reinterpret_cast<const float4*>((const float*)gamma + o * 8 + 4));
      } else {
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g[i]);
        const float2 a0 = __bfloat1622float2(gp[0]), a1 = __bfloat1622float2(gp[1]);
        const float2 a2 = __bfloat1622float2(gp[2]), a3 = __bfloat1622float2(gp[3]);
        g0 = make_float4(a0.x, a0.y, a1.x, a1.y);
        g1 = make_float4(a2.x, a2.y, a3.x, a3.y);
      }
      w.x = pack_bf16(a[i][0].x * g0.x / r, a[i][0].y * g0.y / r);
      w.y = pack_bf16(a[i][0].z * g0.z / r, a[i][0].w * g0.w / r);
      w.z = pack_bf16(a[i][1].x * g1.x / r, a[i][1].y * g1.y / r);
      w.w = pack_bf16(a[i][1].z * g1.z / r, a[i][1].w * g1.w / r);
    }
    *reinterpret_cast<uint4*>(b_chunk(sh.U, kbl, m, o & 7)) = w;
  }
  // token rows that no thread group owns (TPT = 32 covers 8 tokens of the 16 columns)
  if (TPT == 32) {
    const int ch = wt & 7, mm = 8 + ((wt >> 3) & 7);
    for (int kbl = wt >> 6; kbl < nkb; kbl += 4)
      *reinterpret_cast<uint4*>(b_chunk(sh.U, kbl, mm, ch)) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// The k blocks [kb0, kb0 + nkb) of a bf16 activation [16][ld] that an earlier phase wrote.
__device__ __forceinline__ void copy_operand(const DlParams& p, DlShared& sh, const bf16* src,
                                             int ld, int K, int kb0, int nkb, int wt) {
  const int ch = wt & 7, m = (wt >> 3) & 15, kb_first = wt >> 7;
  const bool live = m < p.M;
  for (int kbl = kb_first; kbl < nkb; kbl += 8) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = min((kb0 + min(kbl + 2 * u, nkb - 1)) * BK + ch * 8, K - 8);
      v[u] = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)(live ? m : 0) * ld + k));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int kk = kbl + 2 * u;
      if (kk >= nkb) break;
      const int k = (kb0 + kk) * BK + ch * 8;
      *reinterpret_cast<uint4*>(b_chunk(sh.U, kk, m, ch)) =
          (live && k < K) ? v[u] : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

__device__ __forceinline__ void operand_ready(DlShared& sh, int wt) {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  named_bar(1, DL_WORKERS);
  if (wt == 0) mbar_arrive(sh.b_ready);
}

// ----------------------------------------------------------------------------- attention
// One (request, kv head, chunk of 16 query heads, split of the keys) on the first 128 workers.
// q and the new k are rotated here from the q/k/v product's partial sums; the item whose keys
// include the new token writes its k and v to the cache page before it reads that range.
__device__ __noinline__ void attention_item(const DlParams& p, const DlLayer& L, DlShared& sh, int item,
                               int tid) {
  const int S = p.attn_splits, chunks = p.attn_chunks, G = p.NH / p.NKV;
  const int split = item % S;
  int rest = item / S;
  const int chunk = rest % chunks;
  rest /= chunks;
  const int kvh = rest % p.NKV, b = rest / p.NKV;
  const int h0 = kvh * G + chunk * 16, nrows = min(16, G - chunk * 16);
  const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int pos = p.positions[b];
  const int lo = L.window > 0 ? max(0, pos - L.window + 1) : 0;
  const int nkeys = pos - lo + 1;
  int per = (nkeys + S - 1) / S;
  per = (per + KT - 1) / KT * KT;
  const int begin = lo + split * per, end = min(pos + 1, begin + per);
  const int ntiles = begin < end ? (end - begin + KT - 1) / KT : 0;
  const int page_size = p.page_size;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
  const size_t tok_stride = (size_t)p.NKV * HD;

  bf16* ks = reinterpret_cast<bf16*>(sh.U);                      // [stages][KT][ROW]
  bf16* vs = ks + DL_ATT_STAGES * KT * ROW;
  bf16* qs = vs + DL_ATT_STAGES * KT * ROW;                      // [16][HD]
  int* stbl = reinterpret_cast<int*>(qs + 16 * HD);
  const int* tbl = p.block_table[L.group] + (size_t)b * p.table_stride[L.group];

  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  if (ntiles > 0) {
    // q (and, in the owner, the new k and v) from the q/k/v product: rotated in fp32, rounded to
    // bf16
    const int half = p.rot >> 1;
    const float* cs = p.rope ? p.rope + (size_t)pos * p.rot : nullptr;
    const bf16* qrow = p.qkv + (size_t)b * p.NQKV;
    auto value = [&](int col) -> float { return __bfloat162float(qrow[col]); };
    for (int i = tid; i < nrows * half; i += NTHREADS) {
      const int r = i / half, j = i - r * half;
      const float a = value((h0 + r) * HD + j), bb = value((h0 + r) * HD + j + half);
      const float c = cs[j], s = cs[half + j];
      qs[r * HD + j] = __float2bfloat16_rn(a * c - bb * s);
      qs[r * HD + j + half] = __float2bfloat16_rn(a * s + bb * c);
    }
    const int tail = HD - p.rot;
    for (int i = tid; i < nrows * tail; i += NTHREADS) {
      const int r = i / tail, j = p.rot + (i - r * tail);
      qs[r * HD + j] = __float2bfloat16_rn(value((h0 + r) * HD + j));
    }
    const bool owner = chunk == 0 && pos >= begin && pos < end && L.write_cache;
    if (owner) {
      const int lp = pos / page_size;
      const size_t slot = (size_t)tbl[lp] * page_size + (pos - lp * page_size);
      bf16* kd = L.kpages + slot * tok_stride + (size_t)kvh * HD;
      bf16* vd = L.vpages + slot * tok_stride + (size_t)kvh * HD;
      const int kc = (p.NH + kvh) * HD, vc = (p.NH + p.NKV + kvh) * HD;
      for (int j = tid; j < half; j += NTHREADS) {
        const float a = value(kc + j), bb = value(kc + j + half);
        const float c = cs[j], s = cs[half + j];
        kd[j] = __float2bfloat16_rn(a * c - bb * s);
        kd[j + half] = __float2bfloat16_rn(a * s + bb * c);
      }
      for (int j = p.rot + tid; j < HD; j += NTHREADS) kd[j] = __float2bfloat16_rn(value(kc + j));
      for (int j = tid; j < HD; j += NTHREADS) vd[j] = qrow[vc + j];
      __threadfence();
    }
    // this split's block-table entries -> shared memory
    int lp_base = 0;
    {
      const int lp0 = begin / page_size, nlp = (end - 1) / page_size - lp0 + 1;
      if (nlp <= p.tbl_cap) {
        for (int i = tid; i < nlp; i += NTHREADS) stbl[i] = tbl[lp0 + i];
        tbl = stbl;
        lp_base = lp0;
      }
    }
    named_bar(2, NTHREADS);
    uint32_t qf[KCH][4];
#pragma unroll
    for (int kc = 0; kc < KCH; ++kc) {
      const int d = kc * 16 + 2 * t;
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(qs + g * HD + d);
      const uint32_t* r1 = reinterpret_cast<const uint32_t*>(qs + (g + 8) * HD + d);
      qf[kc][0] = g < nrows ? r0[0] : 0u;
      qf[kc][1] = g + 8 < nrows ? r1[0] : 0u;
      qf[kc][2] = g < nrows ? r0[4] : 0u;
      qf[kc][3] = g + 8 < nrows ? r1[4] : 0u;
    }
    const int lo2[2] = {begin, begin}, hi2[2] = {end - 1, end - 1};
    load_kv_tiles(ks, vs, L.kpages, L.vpages, tbl, lp_base, begin, begin, end, page_size,
                  page_shift, tok_stride, kvh, tid);
    cp_async_commit();
    for (int it = 0; it < ntiles; ++it) {
      cp_async_wait<0>();
      named_bar(2, NTHREADS);
      const int nxt = it + 1;
      if (nxt < ntiles) {
        const int st = nxt % DL_ATT_STAGES;
        load_kv_tiles(ks + st * KT * ROW, vs + st * KT * ROW, L.kpages, L.vpages, tbl, lp_base,
                      begin + nxt * KT, begin, end, page_size, page_shift, tok_stride, kvh, tid);
      }
      cp_async_commit();
      const int st = it % DL_ATT_STAGES;
      const int col0 = begin + it * KT + warp * 16;
      if (col0 < end) {
        float s[2][4] = {};
        qk_tile<2>(s, qf, ks + st * KT * ROW, warp * 16, lane);
        if (col0 + 16 <= end)
          softmax_update<2, false>(s, o, m, l, col0, lo2, hi2, p.scale_log2, lane);
        else
          softmax_update<2, true>(s, o, m, l, col0, lo2, hi2, p.scale_log2, lane);
        pv_tile<2>(o, s, vs + st * KT * ROW, warp * 16, lane);
      }
    }
    cp_async_wait<0>();
  }
  named_bar(2, NTHREADS);

  // merge the four warps through shared memory (reusing the tile buffers)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  float* so = reinterpret_cast<float*>(sh.U);                    // [4][16][HD]
  float* sm = so + 4 * 16 * HD;                                  // [4][16]
  float* sl = sm + 4 * 16;                                       // [4][16]
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    float* base = so + (warp * 16) * HD + n * 8 + 2 * t;
    base[g * HD] = o[n][0];
    base[g * HD + 1] = o[n][1];
    base[(g + 8) * HD] = o[n][2];
    base[(g + 8) * HD + 1] = o[n][3];
  }
  if (t == 0) {
    sm[warp * 16 + g] = m[0];
    sm[warp * 16 + g + 8] = m[1];
    sl[warp * 16 + g] = l[0];
    sl[warp * 16 + g + 8] = l[1];
  }
  named_bar(2, NTHREADS);
  const size_t out_ld = (size_t)p.NH * HD;
  for (int i = tid; i < nrows * HD; i += NTHREADS) {
    const int r = i / HD, d = i - r * HD;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sm[w * 16 + r]);
    float acc = 0.f, lsum = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float wgt = mm == -INFINITY ? 0.f : exp2f(sm[w * 16 + r] - mm);
      acc += wgt * so[(w * 16 + r) * HD + d];
      lsum += wgt * sl[w * 16 + r];
    }
    const int head = h0 + r;
    if (S == 1) {
      p.attn_out[(size_t)b * out_ld + (size_t)head * HD + d] =
          __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    } else {
      const size_t pi = ((size_t)b * p.NH + head) * S + split;
      p.att_o[pi * HD + d] = acc;
      if (d == 0) {
        p.att_ml[pi * 2] = mm;
        p.att_ml[pi * 2 + 1] = lsum;
      }
    }
  }
  if (S == 1) {
    named_bar(2, NTHREADS);               // the tile buffers are free for the next item
    return;
  }
  // the CTA that finishes this (request, kv head, chunk) last merges the splits in split order
  __threadfence();
  named_bar(2, NTHREADS);
  const unsigned int group = ((unsigned int)b * p.NKV + kvh) * chunks + chunk;
  if (tid == 0) {
    const unsigned int done = atomicAdd(p.counters + group, 1u);
    const int last = done == (unsigned int)S - 1;
    if (last) p.counters[group] = 0;
    *sh.flag = last;
  }
  named_bar(2, NTHREADS);
  if (!*sh.flag) {
    named_bar(2, NTHREADS);
    return;
  }
  __threadfence();
  const int used = min(S, per > 0 ? (nkeys + per - 1) / per : 0);
  float* w = reinterpret_cast<float*>(sh.U);                     // [16][used]: weight of a split
  float* linv = w + 16 * DL_MAX_SPLITS;                          // [16]
  for (int i = tid; i < nrows * used; i += NTHREADS) {
    const int r = i / used, s2 = i - r * used;
    const size_t base = ((size_t)b * p.NH + h0 + r) * S;
    w[r * used + s2] = __ldcg(p.att_ml + (base + s2) * 2);       // the split's maximum for now
  }
  named_bar(2, NTHREADS);
  float wl[DL_MAX_SPLITS];
  if (tid < nrows) {
    const int r = tid;
    const size_t base = ((size_t)b * p.NH + h0 + r) * S;
    float mm = -INFINITY;
    for (int s2 = 0; s2 < used; ++s2) mm = fmaxf(mm, w[r * used + s2]);
    float lsum = 0.f;
    for (int s2 = 0; s2 < used; ++s2) {
      const float ms = w[r * used + s2];
      wl[s2] = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      lsum += wl[s2] * __ldcg(p.att_ml + (base + s2) * 2 + 1);
    }
    linv[r] = lsum > 0.f ? 1.f / lsum : 0.f;
  }
  named_bar(2, NTHREADS);                  // every maximum is read before the weights replace them
  if (tid < nrows)
    for (int s2 = 0; s2 < used; ++s2) w[tid * used + s2] = wl[s2];
  named_bar(2, NTHREADS);
  for (int i = tid; i < nrows * HD; i += NTHREADS) {
    const int r = i / HD, d = i - r * HD;
    const float* src = p.att_o + ((size_t)b * p.NH + h0 + r) * S * HD + d;
    float acc = 0.f;
#pragma unroll 4
    for (int s2 = 0; s2 < used; ++s2) acc += w[r * used + s2] * __ldcg(src + (size_t)s2 * HD);
    p.attn_out[(size_t)b * out_ld + (size_t)(h0 + r) * HD + d] = __float2bfloat16_rn(acc * linv[r]);
  }
  named_bar(2, NTHREADS);
}

// ----------------------------------------------------------------------------- epilogues
// Worker warp ww drains TMEM lanes 32 * (warp % 4) .. + 31 (a hardware rule) and the token columns
// 8 * (ww / 4) .. + 7: thread = one weight row, eight tokens.
__device__ __noinline__ void epilogue(const DlParams& p, const DlLayer& L, DlShared& sh,
                                         const DlItem& it, uint32_t tmem, int wt) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q = warp & 3, c0 = ((wt >> 5) >> 2) * 8;
  const int n = it.n0 + q * 32 + lane;
  const DlPhase& ph = p.ph[it.phase];
  float v[8];
  tmem_ld8(tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)c0, v);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  if (it.phase == 2) {                                   // gate/up: rows (gate_i, up_i) interleaved
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
      if (!(lane & 1) && n + 1 < ph.N && c0 + j < p.M)
        p.z[(size_t)(c0 + j) * p.I + (n >> 1)] = __float2bfloat16_rn(dl_silu_mul(v[j], other));
    }
    return;
  }
  // q/k/v (+ bias, rounded to bf16 for attention) and the output and down products (added to the
  // residual).  A split product parks its partial sums in the workspace; the CTA that finishes a
  // tile last adds them up in split order.
  const float* bias = L.bias[it.phase];
  const float bv = (bias && n < ph.N) ? __ldg(bias + n) : 0.f;
  float* ws = it.phase == 0 ? p.ws_qkv : p.ws_red;
  float acc[8];
  if (ph.S > 1) {
    if (n < ph.N) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (c0 + j < p.M) ws[((size_t)it.s * DL_MAX_TOKENS + c0 + j) * ph.N + n] = v[j];
    }
    __threadfence();
    named_bar(1, DL_WORKERS);
    if (wt == 0) {
      const int slot = it.phase == 0 ? 0 : it.phase == 1 ? 1 : 2;
      unsigned int* cnt = p.counters + 4096 + slot * 1024 + it.r;
      const unsigned int done = atomicAdd(cnt, 1u);
      const int last = done == (unsigned int)ph.S - 1;
      if (last) *cnt = 0;
      *sh.flag = last;
    }
    named_bar(1, DL_WORKERS);
    if (!*sh.flag) return;
    __threadfence();
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    // Loads without branches (indices are clamped, what a clamped load brings is dropped), eight
    // splits issued together; the additions stay in split order.
    const int nn = min(n, ph.N - 1);
    for (int s0 = 0; s0 < ph.S; s0 += 8) {
      float t[8][8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int su = min(s0 + u, ph.S - 1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int tok = min(c0 + j, p.M - 1);
          t[u][j] = __ldcg(ws + ((size_t)su * DL_MAX_TOKENS + tok) * ph.N + nn);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const bool on = s0 + u < ph.S;
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += on ? t[u][j] : 0.f;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = v[j];
  }
  if (n >= ph.N) return;
  if (it.phase == 0) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < p.M)
        p.qkv[(size_t)(c0 + j) * ph.N + n] = __float2bfloat16_rn(acc[j] + bv);
  } else {
    float old[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      old[j] = __ldcg(p.h + (size_t)min(c0 + j, p.M - 1) * p.H + n);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (c0 + j < p.M) p.h[(size_t)(c0 + j) * p.H + n] = old[j] + (acc[j] + bv);
  }
}

// ----------------------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(DL_THREADS, 1) decode_layers_kernel(const DlParams p) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ int s_dead, s_issued, s_flag;
  __shared__ float s_rms[DL_MAX_TOKENS];
  DlShared sh;
  sh.ring = (unsigned char*)(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  sh.U = sh.ring + (size_t)p.stages * DL_A_BYTES;
  sh.full = (uint64_t*)(sh.U + p.u_bytes);
  sh.empty = sh.full + p.stages;
  sh.b_ready = sh.empty + p.stages;
  sh.acc_full = sh.b_ready + 1;
  sh.tmem_slot = (uint32_t*)(sh.acc_full + 1);
  sh.dead = &s_dead;
  sh.issued = &s_issued;
  sh.flag = &s_flag;
  sh.rms = s_rms;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(sh.full + s, 1);
      mbar_init(sh.empty + s, 1);
    }
    mbar_init(sh.b_ready, 1);
    mbar_init(sh.acc_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_dead = 0;
    s_issued = 0;
    s_flag = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(sh.tmem_slot)), "r"(32u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *sh.tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ weight producer
    if (lane == 0) {
      DlItemIter iter;
      DlItem it;
      int cnt = 0;
      while (!*sh.dead && iter.next(p, cta, ncta, it)) {
        const CUtensorMap* map = &p.layers[it.layer].w[it.phase];
        for (int kb = it.kb0; kb < it.kb0 + it.nkb; ++kb, ++cnt) {
          const int s = cnt % p.stages;
          if (cnt >= p.stages && !mbar_wait(sh.empty + s, ((cnt / p.stages) & 1) ^ 1, p.err, 21)) {
            *sh.dead = 1;
            break;
          }
          if (*sh.dead) break;
          mbar_expect_tx(sh.full + s, DL_A_BYTES);
          tma_load_2d(sh.ring + (size_t)s * DL_A_BYTES, map, sh.full + s, kb * BK, it.n0);
          *sh.issued = cnt + 1;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(DL_BN);
      DlItemIter iter;
      DlItem it;
      int cnt = 0, items = 0;
      bool ok = true;
      while (ok && !*sh.dead && iter.next(p, cta, ncta, it)) {
        ok = mbar_wait(sh.b_ready, items & 1, p.err, 22);     // operand written, TMEM drained
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int i = 0; i < it.nkb; ++i, ++cnt) {
          const int s = cnt % p.stages;
          ok = mbar_wait(sh.full + s, (cnt / p.stages) & 1, p.err, 23);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t ad = umma_desc(smem_u32(sh.ring + (size_t)s * DL_A_BYTES));
          const uint64_t bd = umma_desc(smem_u32(sh.U + (size_t)i * DL_B_BYTES));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(tmem, ad + (uint64_t)(k * UMMA_K * 2 >> 4), bd + (uint64_t)(k * UMMA_K * 2 >> 4),
                 idesc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(sh.empty + s);
        }
        if (ok) umma_commit(sh.acc_full);
        ++items;
      }
      if (!ok) *sh.dead = 1;
      if (*sh.dead) {
        // copies that were asked for still land: wait for them (bounded) before leaving
        const int issued = *sh.issued;
        for (; cnt < issued; ++cnt)
          if (!mbar_wait(sh.full + cnt % p.stages, (cnt / p.stages) & 1, nullptr, 0)) break;
      }
    }
  } else {
    // ------------------------------------------------------------------ workers
    const int wt = threadIdx.x - 64;
    unsigned int epoch = 0;
    bool ok = true;
    if (wt == 0) dl_stamp(p, 0);
    if (p.emb) {                                           // the residual starts as the embedding
      const int per_row = p.H / 8;
      for (int i = cta * DL_WORKERS + wt; i < p.M * per_row; i += ncta * DL_WORKERS) {
        const int m = i / per_row, c = (i - m * per_row) * 8;
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(
            p.emb + (size_t)p.token_ids[m] * p.H + c));
        const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a0 = __bfloat1622float2(e[0]), a1 = __bfloat1622float2(e[1]);
        const float2 a2 = __bfloat1622float2(e[2]), a3 = __bfloat1622float2(e[3]);
        float4* dst = reinterpret_cast<float4*>(p.h + (size_t)m * p.H + c);
        dst[0] = make_float4(a0.x, a0.y, a1.x, a1.y);
        dst[1] = make_float4(a2.x, a2.y, a3.x, a3.y);
      }
      ok = grid_barrier(p, sh, epoch, wt);
    }
    if (wt == 0) dl_stamp(p, 1);
    DlItemIter iter;
    DlItem it;
    bool have = iter.next(p, cta, ncta, it);
    int items = 0;
    constexpr int gemm_phase[5] = {0, -1, 1, 2, 3};
    for (int layer = 0; ok && layer < p.num_layers; ++layer) {
      const DlLayer& L = p.layers[layer];
      for (int phase = 0; ok && phase < 5; ++phase) {
        if (p.stop_layer >= 0 && (layer > p.stop_layer ||
                                  (layer == p.stop_layer && phase > p.stop_phase))) {
          ok = false;                                       // asked to stop here: not an error
          break;
        }
        if (phase == PH_ATT) {
          if (wt < NTHREADS)
            for (int a = cta; a < p.attn_items; a += ncta) attention_item(p, L, sh, a, wt);
        } else {
          const int gp = gemm_phase[phase];
          bool normed = false;
          while (ok && have && it.layer == layer && it.phase == gp) {
            if (gp == 0 || gp == 2) {
              const int which = gp == 0 ? 0 : 1;
              const int octets = ((p.H >> 3) + 7) & ~7;      // whole k blocks are written
              const void* gm = L.gamma[which];
              const int gf = L.gamma_f32[which];
              const float eps = L.eps[which];
              if (p.M <= 8 && octets <= 32 * 6) {
                build_normed_once<32, 6>(p, sh, gm, gf, eps, it.kb0, it.nkb, wt);
              } else if (p.M <= 8 && octets <= 32 * DL_ROW_OCTETS) {
                build_normed_once<32, DL_ROW_OCTETS>(p, sh, gm, gf, eps, it.kb0, it.nkb, wt);
              } else if (octets <= 16 * 6) {
                build_normed_once<16, 6>(p, sh, gm, gf, eps, it.kb0, it.nkb, wt);
              } else if (octets <= 16 * DL_ROW_OCTETS) {
                build_normed_once<16, DL_ROW_OCTETS>(p, sh, gm, gf, eps, it.kb0, it.nkb, wt);
              } else {
                if (!normed) {
                  row_rms(p, sh, L.eps[which], wt);
                  normed = true;
                }
                build_normed(p, sh, L.gamma[which], L.gamma_f32[which], it.kb0, it.nkb, wt);
              }
            } else if (gp == 1) {
              copy_operand(p, sh, p.attn_out, p.NH * HD, p.NH * HD, it.kb0, it.nkb, wt);
            } else {
              copy_operand(p, sh, p.z, p.I, p.I, it.kb0, it.nkb, wt);
            }
            operand_ready(sh, wt);
            if (wt == 0 && !mbar_wait(sh.acc_full, items & 1, p.err, 24)) *sh.dead = 1;
            named_bar(1, DL_WORKERS);
            ++items;
            if (*sh.dead) {
              ok = false;
              break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            epilogue(p, L, sh, it, tmem, wt);
            have = iter.next(p, cta, ncta, it);
          }
        }
        if (wt == 0) dl_stamp(p, 2 + (layer * 5 + phase) * 2);
        if (ok) ok = grid_barrier(p, sh, epoch, wt);
        if (wt == 0) dl_stamp(p, 3 + (layer * 5 + phase) * 2);
      }
    }
    // a worker that leaves early lets the MMA issuer go too
    if (*sh.dead && wt == 0) mbar_arrive(sh.b_ready);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(32u)
                 : "memory");
}

// ----------------------------------------------------------------------------- host side
struct DlPlan {
  DlParams params;
  DlLayer* host_layers;
  int num_sms;
  size_t smem;
};

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

static void plan_phase(DlPhase& ph, int N, int K, int ncta, int max_kb, int off, bool may_split) {
  ph.N = N;
  ph.KB = ceil_div(K, BK);
  const int tiles = ceil_div(N, BM);
  int S = may_split ? ncta / tiles : 1;
  S = S < 1 ? 1 : S > DL_MAX_SPLITS ? DL_MAX_SPLITS : S > ph.KB ? ph.KB : S;
  ph.per = ceil_div(ph.KB, S);
  while (ph.per > max_kb && may_split) ph.per = max_kb;
  ph.S = ceil_div(ph.KB, ph.per);
  ph.off = off;
  ph.items = tiles * ph.S;
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_dl_head_dim() { return HD; }
GF_EXPORT int gf_dl_layer_bytes() { return (int)sizeof(DlLayer); }
GF_EXPORT int gf_dl_max_tokens() { return DL_MAX_TOKENS; }

// A plan for `num_layers` layers of one shape.  Returns null (and a code in *status) if the shape
// is not served: 1 sizes, 2 shared memory, 3 device.
GF_EXPORT void* gf_dl_create(int num_layers, int H, int NH, int NKV, int I, int page_size, int rot,
                             float scale, int device, int* status) {
  *status = 1;
  const int NQKV = (NH + 2 * NKV) * HD;
  if (num_layers < 1 || H % 8 || I % 8 || NH % NKV || rot % 2 || rot > HD || page_size < 1) return nullptr;
  if (ceil_div(H, BM) > 1024 || NH * HD % 8) return nullptr;
  *status = 3;
  int num_sms = 0, max_smem = 0;
  if (cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
      cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess)
    return nullptr;
  int coop = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, device);
  if (!coop) return nullptr;
  *status = 2;
  const int tbl_cap = 1024;
  const size_t att_bytes = (size_t)DL_ATT_STAGES * 2 * KT * ROW * 2 + 16 * HD * 2 + tbl_cap * 4;
  const size_t fixed = 2048;                              // alignment slack and barriers
  const size_t reserve = fixed + 4096;                    // and room for static shared memory
  // the unsplit gate/up product needs the whole normalised row as its operand
  const int kb_h = ceil_div(H, BK);
  size_t u = (size_t)kb_h * DL_B_BYTES;
  if (u < att_bytes) u = att_bytes;
  u = (u + 1023) / 1024 * 1024;
  if (u + reserve + 3 * DL_A_BYTES > (size_t)max_smem) return nullptr;
  int stages = (int)(((size_t)max_smem - reserve - u) / DL_A_BYTES);
  if (stages > 32) stages = 32;
  const int max_kb = (int)(u / DL_B_BYTES);

  auto* plan = new DlPlan();
  DlParams& p = plan->params;
  memset(&p, 0, sizeof(p));
  p.num_layers = num_layers;
  p.H = H, p.NH = NH, p.NKV = NKV, p.I = I, p.NQKV = NQKV, p.page_size = page_size, p.rot = rot;
  p.scale_log2 = scale * LOG2E;
  int off = 0;
  plan_phase(p.ph[0], NQKV, H, num_sms, max_kb, off, true);
  off = (off + p.ph[0].items) % num_sms;
  plan_phase(p.ph[1], H, NH * HD, num_sms, max_kb, off, true);
  off = (off + p.ph[1].items) % num_sms;
  plan_phase(p.ph[2], 2 * I, H, num_sms, max_kb, off, false);
  off = (off + p.ph[2].items) % num_sms;
  plan_phase(p.ph[3], H, I, num_sms, max_kb, off, true);
  for (int i = 0; i < 4; ++i)
    if (p.ph[i].per > max_kb || p.ph[i].S > DL_MAX_SPLITS) {
      delete plan;
      return nullptr;
    }
  p.attn_chunks = ceil_div(NH / NKV, 16);
  p.stages = stages;
  p.u_bytes = (uint32_t)u;
  p.tbl_cap = tbl_cap;
  p.stop_layer = -1, p.stop_phase = -1;
  plan->num_sms = num_sms;
  plan->smem = fixed + u + (size_t)stages * DL_A_BYTES;
  plan->host_layers = new DlLayer[num_layers];
  memset(plan->host_layers, 0, sizeof(DlLayer) * num_layers);
  cudaError_t e = cudaFuncSetAttribute(decode_layers_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan->smem);
  int resident = 0;
  if (e == cudaSuccess)
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, decode_layers_kernel, DL_THREADS,
                                                      plan->smem);
  if (e != cudaSuccess || resident < 1) {
    delete[] plan->host_layers;
    delete plan;
    return nullptr;
  }
  *status = 0;
  return plan;
}

GF_EXPORT void gf_dl_destroy(void* handle) {
  auto* plan = (DlPlan*)handle;
  if (!plan) return;
  delete[] plan->host_layers;
  delete plan;
}

// Sizes (in elements) of the buffers a caller provides: h, ws_qkv, att_o, att_ml, attn_out, ws_red,
// z, counters, qkv; and the schedule (splits of the four products, ring depth) for reports.
GF_EXPORT void gf_dl_sizes(void* handle, long long* out, int* sched) {
  const DlParams& p = ((DlPlan*)handle)->params;
  out[0] = (long long)DL_MAX_TOKENS * p.H;
  out[1] = (long long)p.ph[0].S * DL_MAX_TOKENS * p.NQKV;
  out[2] = (long long)DL_MAX_TOKENS * p.NH * DL_MAX_SPLITS * HD;
  out[3] = (long long)DL_MAX_TOKENS * p.NH * DL_MAX_SPLITS * 2;
  out[4] = (long long)DL_MAX_TOKENS * p.NH * HD;
  const int smax = p.ph[1].S > p.ph[3].S ? p.ph[1].S : p.ph[3].S;
  out[5] = (long long)smax * DL_MAX_TOKENS * p.H;
  out[6] = (long long)DL_MAX_TOKENS * p.I;
  out[7] = 4096 + 3072;
  out[8] = (long long)DL_MAX_TOKENS * p.NQKV;
  for (int i = 0; i < 4; ++i) sched[i] = p.ph[i].S;
  sched[4] = p.stages;
  sched[5] = ((DlPlan*)handle)->num_sms;
  sched[6] = (int)((DlPlan*)handle)->smem;
}

GF_EXPORT int gf_dl_set_layer(void* handle, int i, const void* w_qkv, const void* w_o,
                              const void* w_gu, const void* w_down, const float* b_qkv,
                              const float* b_o, const float* b_down, const void* gamma1,
                              int gamma1_f32, float eps1, const void* gamma2, int gamma2_f32,
                              float eps2) {
  auto* plan = (DlPlan*)handle;
  const DlParams& p = plan->params;
  if (i < 0 || i >= p.num_layers) return -1;
  DlLayer& L = plan->host_layers[i];
  const int ao = p.NH * HD;
  if (!make_map(&L.w[0], w_qkv, p.NQKV, p.H, p.H, BM) || !make_map(&L.w[1], w_o, p.H, ao, ao, BM) ||
      !make_map(&L.w[2], w_gu, 2 * p.I, p.H, p.H, BM) || !make_map(&L.w[3], w_down, p.H, p.I, p.I, BM))
    return -4;
  L.bias[0] = b_qkv, L.bias[1] = b_o, L.bias[2] = nullptr, L.bias[3] = b_down;
  L.gamma[0] = gamma1, L.gamma[1] = gamma2;
  L.gamma_f32[0] = gamma1_f32, L.gamma_f32[1] = gamma2_f32;
  L.eps[0] = eps1, L.eps[1] = eps2;
  return 0;
}

GF_EXPORT int gf_dl_set_cache(void* handle, int i, void* kpages, void* vpages, int group,
                              int window, int write) {
  auto* plan = (DlPlan*)handle;
  if (i < 0 || i >= plan->params.num_layers || group < 0 || group >= DL_MAX_GROUPS) return -1;
  DlLayer& L = plan->host_layers[i];
  L.kpages = (bf16*)kpages, L.vpages = (bf16*)vpages;
  L.group = group;
  L.window = window, L.write_cache = write;
  return 0;
}

// Copy the layer descriptions to `dev_layers` (gf_dl_layer_bytes() * layers bytes of device memory).
GF_EXPORT int gf_dl_upload(void* handle, void* dev_layers, void* stream) {
  auto* plan = (DlPlan*)handle;
  plan->params.layers = (const DlLayer*)dev_layers;
  cudaError_t e = cudaMemcpyAsync(dev_layers, plan->host_layers,
                                  sizeof(DlLayer) * plan->params.num_layers,
                                  cudaMemcpyHostToDevice, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  return (int)e;
}

// One step: M tokens (requests), one each.  `bufs`: h, ws_qkv, att_o, att_ml, attn_out, ws_red, z,
// counters (zero before the first call), qkv, in the sizes gf_dl_sizes gives.  `bar` is one word.
// `tables[g]`: the block table of cache group g for this step, rows in the order of the tokens.
GF_EXPORT int gf_dl_run(void* handle, int M, const int* token_ids, const void* emb,
                        const int* positions, const float* rope, const void* const* tables,
                        const int* table_strides, int num_tables, void* const* bufs,
                        unsigned int* bar, int* err, int stop_layer, int stop_phase,
                        unsigned long long* stamps, void* stream) {
  auto* plan = (DlPlan*)handle;
  if (M < 1 || M > DL_MAX_TOKENS) return -2;
  DlParams p = plan->params;
  if (!p.layers) return -3;
  p.M = M;
  p.token_ids = token_ids, p.emb = (const bf16*)emb, p.positions = positions, p.rope = rope;
  p.h = (float*)bufs[0], p.ws_qkv = (float*)bufs[1], p.att_o = (float*)bufs[2];
  p.att_ml = (float*)bufs[3], p.attn_out = (bf16*)bufs[4], p.ws_red = (float*)bufs[5];
  p.z = (bf16*)bufs[6], p.counters = (unsigned int*)bufs[7], p.qkv = (bf16*)bufs[8];
  p.bar = bar, p.err = err;
  p.stamps = stamps;
  if (num_tables < 1 || num_tables > DL_MAX_GROUPS) return -2;
  for (int g = 0; g < DL_MAX_GROUPS; ++g) {
    p.block_table[g] = (const int*)tables[g < num_tables ? g : 0];
    p.table_stride[g] = table_strides[g < num_tables ? g : 0];
  }
  p.stop_layer = stop_layer, p.stop_phase = stop_phase;
  const int groups = M * p.NKV * p.attn_chunks;
  int S = plan->num_sms / groups;
  S = S < 1 ? 1 : S > 8 ? 8 : S;
  p.attn_splits = S;
  p.attn_items = groups * S;
  if (groups > 4096) return -2;
  auto st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(bar, 0, sizeof(unsigned int), st);
  if (e != cudaSuccess) return (int)e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(plan->num_sms);
  cfg.blockDim = dim3(DL_THREADS);
  cfg.dynamicSmemBytes = plan->smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, decode_layers_kernel, p);
}
