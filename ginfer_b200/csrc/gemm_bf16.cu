// bf16 matrix products on the 5th-generation tensor cores: out[M, N] = x[M, K] * W[N, K]^T with fp32
// accumulation in tensor memory, operands staged in shared memory by TMA.
//
// The weight matrix is the A operand: a CTA owns 128 rows of W (TMEM lanes) and BN tokens (TMEM
// columns, BN = 16 .. 256), so the same kernel serves prefill (BN = 256) and decode, where a batch
// of 8 .. 64 tokens would waste a 128-row tile if tokens were the A operand.  Both operands are
// K-major in global memory (x [M, K] and W [N, K] as Hugging Face stores it), so no transposition
// is needed; TMA writes 128-byte-swizzled [rows][64] tiles that the UMMA descriptors name directly.
//
// Roles (192 threads): warp 0 issues TMA loads through a ring of STAGES stages; warp 1 allocates
// tensor memory and issues tcgen05.mma (one thread), releasing stages with tcgen05.commit; warps
// 2..5 read the accumulator back with tcgen05.ld and run the epilogue:
//   EPI_STORE  out = acc (+ bias[n]) as bf16 or fp32
//   EPI_SILU   W rows are interleaved (gate_i, up_i): out[m, i] = silu(bf16(gate)) * bf16(up)
//   EPI_RESID  s = resid + acc (+ bias[n]) in fp32, the new residual stream; beside it
//              bf16(s * gamma[n]) (the operand of the product behind the next RMS norm) and, per
//              token, this CTA's share of sum_n s^2
// An RMS normalisation in front of a product costs no kernel of its own: the product before it
// leaves bf16(s * gamma) and partial sums of squares (EPI_RESID), and the product behind it
// multiplies its accumulator by 1 / rms[token] = rsqrt(sum of the partials / K + eps) (`in_sumsq`;
// every epilogue takes it), since (s gamma / rms) W^T = (s gamma) W^T / rms.
// Products whose tiles alone would leave most SMs idle (the small-N products of a decode step) split
// the K range, deterministically, in one of two ways.  Cluster mode (split_k 2, 4, 8 or 12): the
// splits of a tile form a thread-block cluster and each CTA sums a band of the tile's rows over all
// peers, in rank order, and runs the epilogue for it.  Where a split's K range leaves stages of the
// ring unused (the q/k/v and output products of decode steps) the partials are pushed: every thread
// sends its row's partial sums into the band owner's shared memory (st.async, counted by the
// owner's mbarrier), the owner waits for the bytes, and nobody waits for a barrier of the cluster
// after the set-up; in a decode step of 4 layers at the 1.5B shape 258.4 us against 260.4.
// Otherwise they are pulled: every CTA parks its partial tile in its own shared memory, and after
// a cluster barrier the owners read their bands through distributed shared memory (and a second
// barrier keeps everyone until the reads are done).  Workspace mode (any split_k): the partials
// go to global memory and the split that finishes a tile last (counted with an atomic it resets)
// sums them in split order.
//
// The reference calls cuBLASLt for every product (ginfer/core/op/kernels/cuda/gemm_kernel/
// gemm_kernel.cu:93-156, bias in the epilogue :112-121, fp32 compute :100) and has a separate
// SwiGLU kernel (swiglu_kernel.cu:6-31).
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records an error code in
// *err and leaves its loop; all roles then meet at the final barrier, the CTA waits (bounded again)
// for those of its own copies that nobody consumed, and tensor memory is freed.  A build with
// -DGF_TEST_SKIP_STAGE (and a small -DGF_SPIN_LIMIT) leaves out the loads of one K block so that a
// test can watch this happen: the MMA issuer's wait runs out, the kernel returns, *err says 2.
#include "tc_common.cuh"

namespace gf {

constexpr int NTHREADS = 192;
constexpr int EPI_STORE = 0, EPI_SILU = 2, EPI_RESID = 3;

struct GemmExtra {
  // consumer of a deferred RMS normalisation: scale[m] = rsqrt(sum_p in_sumsq[p][m] * inv_k + eps)
  const float* in_sumsq;     // [in_parts][ss_ld] or null
  int in_parts;
  int ss_ld;
  float in_eps;
  float inv_k;
  // EPI_RESID
  const float* resid;        // [M][ldo]
  bf16* out_scaled;          // [M][ldo] or null
  const void* gamma;         // [N], bf16 or fp32
  int gamma_f32;
  float* out_sumsq;          // [parts][ss_ld]; part = tile of rows (* splits + split)
};
constexpr int kMaxTiles = 1 << 16;
__device__ unsigned int g_tile_done[kMaxTiles];

#ifdef GF_STAMPS
// Debug build: every CTA records when it started, issued its prefetch, was released by the kernel
// ahead, had its accumulator and left (globaltimer, ns), for reading back on the host.
constexpr unsigned int kStampCap = 1 << 15;
__device__ unsigned long long g_stamps[kStampCap * 8];
__device__ unsigned int g_stamp_next;
__shared__ unsigned int stamp_slot;
__device__ __forceinline__ unsigned long long gtime() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define GF_STAMP(i) (g_stamps[(size_t)stamp_slot * 8 + (i)] = gtime())
#else
#define GF_STAMP(i) ((void)0)
#endif

__host__ __device__ constexpr int stages_for(int bn) {
  // Ring of (16 KB + bn * 128 B) stages.  Small token tiles (decode) stay within ~110 KB so that
  // two CTAs, of this product or of the next one in the stream, share an SM; large ones take
  // ~200 KB.  At most 8 stages.
  const int budget = bn <= 64 ? 110 * 1024 : 200 * 1024;
  const int n = budget / (BM * BK * 2 + bn * BK * 2);
  return n > 8 ? 8 : n;
}

template <typename OUT> __device__ __forceinline__ void store_out(OUT* p, float v);
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) {
  *p = __float2bfloat16_rn(v);
}
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }

__device__ __forceinline__ float gamma_at(const GemmExtra& ex, int n) {
  return ex.gamma_f32 ? reinterpret_cast<const float*>(ex.gamma)[n]
                      : __bfloat162float(reinterpret_cast<const bf16*>(ex.gamma)[n]);
}
__device__ __forceinline__ float silu_mul(float g, float u) {
  const float gg = __bfloat162float(__float2bfloat16_rn(g));
  const float uu = __bfloat162float(__float2bfloat16_rn(u));
  return gg * (1.0f / (1.0f + expf(-gg))) * uu;
}

// Epilogue of 16 accumulator columns (tokens m_base .. m_base + 15) of W row n for one thread.
// `scale`: per-token factors of a deferred normalisation (shared memory, indexed from the tile's
// first token) or null.  EPI_RESID: sq[j] receives the square of what was stored (0 where nothing).
template <int EPI, typename OUT>
__device__ __forceinline__ void epilogue16(float (&v)[16], OUT* __restrict__ out, int ldo,
                                           const float* __restrict__ bias, int n, int m_base,
                                           int M, int N, int lane, const float* scale,
                                           const GemmExtra& ex, float (&sq)[16]) {
  if (scale) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] *= scale[j];
  }
  if (EPI == EPI_STORE) {
    const float b = (bias && n < N) ? bias[n] : 0.f;
    if (n < N) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (m_base + j < M) store_out<OUT>(out + (size_t)(m_base + j) * ldo + n, v[j] + b);
    }
  } else if (EPI == EPI_RESID) {
    const float b = (bias && n < N) ? bias[n] : 0.f;
    const float g = (ex.out_scaled && n < N) ? gamma_at(ex, n) : 0.f;
    // the residual's loads first and unguarded (clamped): guarded ones would wait in line
    float r[16];
    const int nc = min(n, N - 1);
#pragma unroll
    for (int j = 0; j < 16; ++j)
      r[j] = __ldcg(ex.resid + (size_t)min(m_base + j, M - 1) * ldo + nc);
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      sq[j] = 0.f;
      if (n < N && m_base + j < M) {
        const size_t at = (size_t)(m_base + j) * ldo + n;
        const float h = r[j] + (v[j] + b);
        store_out<OUT>(out + at, h);
        if (ex.out_scaled) ex.out_scaled[at] = __float2bfloat16_rn(h * g);
        sq[j] = h * h;
      }
    }
  } else {
    // rows come in pairs (gate, up) on adjacent lanes; each lane finishes every other token
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
      if ((j & 1) == (lane & 1)) {
        const float g = (lane & 1) ? other : v[j], u = (lane & 1) ? v[j] : other;
        const int pair = n >> 1;
        if ((n | 1) < N && m_base + j < M)
          store_out<OUT>(out + (size_t)(m_base + j) * ldo + pair, silu_mul(g, u));
      }
    }
  }
}

// Cluster split-K.  Every CTA parks its partial tile in its own shared memory, token by token:
// red[token][RED_LD] with the tile's 128 rows side by side.  After the cluster's barrier the
// first 128 / band CTAs each sum a band of rows (16 at least: a 32-byte sector of bf16 output, so
// that what they store are whole sectors, which the next kernel's loads need not complete from
// memory) over all SPLIT peers, read through distributed shared memory; a thread takes four
// neighbouring rows of one token.  The peers' loads are issued together and the additions stay in
// rank order.  `scale`: per-token factors in this CTA's shared memory or null.  EPI_RESID: `sqs`
// (shared memory behind the parked tile, band / 4 * BN floats) takes the squares, which one thread
// per token adds up in row order into this CTA's part of out_sumsq (parts of idle CTAs are 0).
constexpr int RED_LD = BM + 4;
template <int SPLIT> struct Band {
  static constexpr int rows = (BM / SPLIT + 15) / 16 * 16 < 16 ? 16 : (BM / SPLIT + 15) / 16 * 16;
};

__device__ __forceinline__ void store4(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void store4(bf16* p, const float (&v)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 w;
  w.x = *reinterpret_cast<uint32_t*>(&a);
  w.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = w;
}

// Where the partial of (chunk of 16 tokens, split `src`, row of the band, token) lies in a band
// owner's receive area, in floats.  A sender writes four tokens at a time; the pieces of a row are
// swapped by the row's quad so that readers of one token in neighbouring quads meet no bank twice.
__device__ __forceinline__ int recv_at(int chunk, int src, int row, int tok16, int split, int band) {
  return ((chunk * split + src) * band + row) * 16 + ((((tok16 >> 2) ^ (row >> 2)) & 3) << 2) +
         (tok16 & 3);
}

// PUSH = false: `red` is the parked tile's address (see above), the peers are read after the
// cluster's barrier, all NTHREADS threads work.  PUSH = true: the peers have sent their rows of
// this CTA's band into `recv` (recv_at), counted by `recv_bar`; the 128 epilogue threads wait
// for it and work, and nothing of a peer is touched.
template <int BN, int EPI, typename OUT, int SPLIT, bool PUSH>
__device__ __forceinline__ void cluster_reduce(uint32_t red, const float* recv, uint64_t* recv_bar,
                                               int* err, const float* __restrict__ bias,
                                               OUT* __restrict__ out, int ldo, int M, int N,
                                               int n0, int m0, const float* scale,
                                               const GemmExtra& ex, float* sqs) {
  const int rank = (int)cluster_rank();
  constexpr int band = Band<SPLIT>::rows;
  constexpr int QUADS = band / 4;                     // a unit of work: four rows of one token
  constexpr int UNITS = QUADS * BN;
  constexpr int GROUP = PUSH ? 128 : NTHREADS;
  const int uid = PUSH ? (int)threadIdx.x - 64 : (int)threadIdx.x;
  const bool active = rank * band < BM;
  // vector stores need four rows that exist and an aligned row of the output
  const bool vec = (ldo & 3) == 0 && (N & 3) == 0;
  // EPI_RESID: the residual of this thread's first unit (the only one when the band's units are
  // no more than the threads, as in decode steps) is asked for before the partials are waited for
  float rs0[4] = {0.f, 0.f, 0.f, 0.f};
  if (EPI == EPI_RESID && active && uid < UNITS) {
    const int tok = uid / QUADS, n = n0 + rank * band + (uid % QUADS) * 4;
    const float* src = ex.resid + (size_t)min(m0 + tok, M - 1) * ldo;
#pragma unroll
    for (int j = 0; j < 4; ++j) rs0[j] = __ldcg(src + min(n + j, N - 1));
  }
  // the bias of the first unit likewise: it may come from memory, and nothing it waits for
  float b0[4] = {0.f, 0.f, 0.f, 0.f};
  if (EPI != EPI_SILU && bias && active && uid < UNITS) {
    const int n = n0 + rank * band + (uid % QUADS) * 4;
#pragma unroll
    for (int j = 0; j < 4; ++j) b0[j] = __ldg(bias + min(n + j, N - 1));
  }
  bool have = true;
  if (PUSH) {
    if (active) have = mbar_wait(recv_bar, 0, err, 3);
  } else {
    cluster_sync();                                   // every peer's partial tile is parked
  }
  if (active && have) {
    for (int u = uid; u < UNITS; u += GROUP) {
      const int tok = u / QUADS, brow = (u % QUADS) * 4, row = rank * band + brow;
      const int n = n0 + row, m = m0 + tok;
      float hh = 0.f;
      if (m < M && n < N) {
        float4 t[SPLIT];
        if (PUSH) {
          const float* src = recv + recv_at(tok >> 4, 0, brow, tok & 15, SPLIT, band);
#pragma unroll
          for (int p = 0; p < SPLIT; ++p) {
            const float* q = src + p * band * 16;
            t[p] = make_float4(q[0], q[16], q[32], q[48]);
          }
        } else {
#pragma unroll
          for (int p = 0; p < SPLIT; ++p)
            t[p] = ld_dsmem_f4(red + (uint32_t)((tok * RED_LD + row) * 4), p);
        }
        float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int p = 0; p < SPLIT; ++p)
          a4.x += t[p].x, a4.y += t[p].y, a4.z += t[p].z, a4.w += t[p].w;
        float v[4] = {a4.x, a4.y, a4.z, a4.w};
        if (scale) {
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] *= scale[tok];
        }
        if (EPI == EPI_SILU) {
          // rows are (gate, up) pairs: two results
          const int pair = n >> 1;
          const float r0 = silu_mul(v[0], v[1]), r1 = silu_mul(v[2], v[3]);
          OUT* dst = out + (size_t)m * ldo + pair;
          if (n + 1 < N) store_out<OUT>(dst, r0);
          if (n + 3 < N) store_out<OUT>(dst + 1, r1);
        } else {
          if (bias) {
            if (u < GROUP) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] += b0[j];
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] += bias[min(n + j, N - 1)];
            }
          }
          const size_t at = (size_t)m * ldo + n;
          if (EPI == EPI_RESID) {
            float rs[4] = {rs0[0], rs0[1], rs0[2], rs0[3]};
            if (u >= GROUP) {
#pragma unroll
              for (int j = 0; j < 4; ++j) rs[j] = __ldcg(ex.resid + (size_t)m * ldo + min(n + j, N - 1));
            }
            float g[4] = {0.f, 0.f, 0.f, 0.f};
            if (ex.out_scaled) {
#pragma unroll
              for (int j = 0; j < 4; ++j) g[j] = gamma_at(ex, min(n + j, N - 1));
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[j] += rs[j];
              if (n + j < N) hh += v[j] * v[j];
              g[j] *= v[j];
            }
            if (vec) {
              store4(out + at, v);
              if (ex.out_scaled) store4(ex.out_scaled + at, g);
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (n + j < N) {
                  store_out<OUT>(out + at + j, v[j]);
                  if (ex.out_scaled) ex.out_scaled[at + j] = __float2bfloat16_rn(g[j]);
                }
            }
          } else if (vec) {
            store4(out + at, v);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (n + j < N) store_out<OUT>(out + at + j, v[j]);
          }
        }
      }
      if (EPI == EPI_RESID) sqs[u] = hh;
    }
  }
  if (EPI == EPI_RESID) {
    if (PUSH)
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
    else
      __syncthreads();
    for (int tok = uid; tok < BN; tok += GROUP) {
      float sum = 0.f;
      if (active && have)
        for (int qd = 0; qd < QUADS; ++qd) sum += sqs[tok * QUADS + qd];
      if (m0 + tok < M)
        ex.out_sumsq[(size_t)(blockIdx.x * SPLIT + rank) * ex.ss_ld + m0 + tok] = sum;
    }
  }
}

template <int BN, int EPI, typename OUT>
struct ReduceBySplit {
  template <bool PUSH>
  static __device__ __forceinline__ void run(int split_k, uint32_t red, const float* recv,
                                             uint64_t* recv_bar, int* err, const float* bias,
                                             OUT* out, int ldo, int M, int N, int n0, int m0,
                                             const float* scale, const GemmExtra& ex, float* sqs) {
    if (split_k == 2)
      cluster_reduce<BN, EPI, OUT, 2, PUSH>(red, recv, recv_bar, err, bias, out, ldo, M, N, n0, m0,
                                            scale, ex, sqs);
    else if (split_k == 4)
      cluster_reduce<BN, EPI, OUT, 4, PUSH>(red, recv, recv_bar, err, bias, out, ldo, M, N, n0, m0,
                                            scale, ex, sqs);
    else if (split_k == 8)
      cluster_reduce<BN, EPI, OUT, 8, PUSH>(red, recv, recv_bar, err, bias, out, ldo, M, N, n0, m0,
                                            scale, ex, sqs);
    else
      cluster_reduce<BN, EPI, OUT, 12, PUSH>(red, recv, recv_bar, err, bias, out, ldo, M, N, n0, m0,
                                             scale, ex, sqs);
  }
};

// Rows of a band of a cluster split at run time (Band<SPLIT>::rows).
__host__ __device__ constexpr int band_rows(int split) {
  return (BM / split + 15) / 16 * 16 < 16 ? 16 : (BM / split + 15) / 16 * 16;
}
// Bytes a band owner receives from its cluster (all splits, every chunk of 16 tokens of the tile).
__host__ __device__ constexpr uint32_t recv_bytes(int bn, int split) {
  return (uint32_t)(bn / 16) * split * band_rows(split) * 16 * 4;
}

// Whether a cluster split adds up in push mode: the stages that no split's K range reaches have
// to hold the receive area (and the squares of an EPI_RESID band behind it).
template <int BN, int EPI>
__host__ __device__ constexpr bool push_fits(int K, int split_k) {
  const int per = ((K + BK - 1) / BK + split_k - 1) / split_k;
  const uint32_t stage = BM * BK * 2 + BN * BK * 2;
  const uint32_t need = recv_bytes(BN, split_k) + (EPI == EPI_RESID ? 16u * BN * sizeof(float) : 0u);
  return split_k > 1 && per + (int)((need + stage - 1) / stage) <= stages_for(BN);
}

template <int BN, int EPI, typename OUT, bool CLUSTER, bool PUSH = false>
__global__ void __launch_bounds__(NTHREADS, 4)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const float* __restrict__ bias, OUT* __restrict__ out, int ldo, int M, int N, int K,
               int split_k, float* __restrict__ workspace, int* __restrict__ err,
               const GemmExtra ex) {
  constexpr int STAGES = stages_for(BN);
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * (A_BYTES + B_BYTES));
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* recv_bar = acc_full + 1;                  // counts what the cluster's peers send here
  uint32_t* tmem_slot = (uint32_t*)(recv_bar + 1);
  float* scale_s = (float*)(tmem_slot + 2);           // [BN] factors of a deferred normalisation
  float* sq_s = scale_s + BN;                         // [4][BN] squares per epilogue warp (EPI_RESID)
  __shared__ bool is_last;
  __shared__ int gave_up;                             // a wait of this CTA ran out
  __shared__ int issued_s;                            // K blocks whose loads the producer got to
#ifdef GF_TEST_SKIP_STAGE
  constexpr int kSkipped = 1;                         // the K block whose loads never go out
#else
  constexpr int kSkipped = -1;
#endif

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN, split = blockIdx.z;
  const int nkb_all = (K + BK - 1) / BK;
  const int per = (nkb_all + split_k - 1) / split_k;
  const int kb0 = split * per, kb1 = min(nkb_all, kb0 + per);
  const int nkb = max(0, kb1 - kb0);
  // Cluster split-K in push mode: the stages that no split's K range reaches take what the peers
  // send.
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr bool push = CLUSTER && PUSH;              // (the launcher asked push_fits)
  float* recv = reinterpret_cast<float*>(tiles + (size_t)per * STAGE_BYTES);

  pdl_trigger();
#ifdef GF_STAMPS
  if (threadIdx.x == 0) {
    stamp_slot = atomicAdd(&g_stamp_next, 1u) % kStampCap;
    unsigned int smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    g_stamps[(size_t)stamp_slot * 8 + 0] = ((unsigned long long)N << 32) | (unsigned int)K;
    g_stamps[(size_t)stamp_slot * 8 + 1] =
        ((unsigned long long)smid << 32) | (blockIdx.x << 8) | blockIdx.z;
    GF_STAMP(2);
  }
#endif
  if (threadIdx.x == 0) {
    gave_up = 0;
    issued_s = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(recv_bar, 1);
    if (push && (int)cluster_rank() * band_rows(split_k) < BM) {
      const int live = min(BN, M - m0);
      mbar_expect_tx(recv_bar, (uint32_t)((live + 15) / 16) * split_k * band_rows(split_k) * 64u);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;
  // push mode: nobody sends before every CTA of the cluster has set its barrier up.  The producer
  // asks for its weights first and waits afterwards.
  if (push) {
    cluster_arrive();
    if (warp != 0) cluster_wait();
  }

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the kernel before this one: fill the ring with them first, then
      // wait for that kernel and add the activations to the same stages.
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        if (i == kSkipped) continue;
        mbar_expect_tx(full + i, A_BYTES + B_BYTES);
        tma_load_2d(tiles + i * (A_BYTES + B_BYTES), &tmap_w, full + i, (kb0 + i) * BK, n0);
      }
      GF_STAMP(3);
      pdl_wait();
      GF_STAMP(4);
      for (int i = 0; i < pre; ++i) {
        if (i == kSkipped) continue;
        tma_load_2d(tiles + i * (A_BYTES + B_BYTES) + A_BYTES, &tmap_x, full + i, (kb0 + i) * BK,
                    m0);
      }
      int issued = pre;
      for (int i = pre; i < nkb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(empty + s, ((i / STAGES) & 1) ^ 1, err, 1)) {
          gave_up = 1;
          break;
        }
        mbar_expect_tx(full + s, A_BYTES + B_BYTES);
        unsigned char* a = tiles + s * (A_BYTES + B_BYTES);
        tma_load_2d(a, &tmap_w, full + s, (kb0 + i) * BK, n0);
        tma_load_2d(a + A_BYTES, &tmap_x, full + s, (kb0 + i) * BK, m0);
        issued = i + 1;
      }
      issued_s = issued;
    }
    if (push) {
      __syncwarp();
      cluster_wait();
    }
  } else if (warp == 1) {
    // The whole warp walks through the K blocks; lane 0 issues the products.  The waits for the
    // stages are made AHEAD stages at a time, each by a lane of its own (mbar_wait_lanes): one
    // after the other they cost the issuing thread more than the products of a stage.
    constexpr uint32_t idesc = umma_idesc(BN);
#ifndef GF_MMA_AHEAD
    constexpr int AHEAD = BN <= 64 ? (STAGES >= 6 ? 3 : 2) : 1;
#else
    constexpr int AHEAD = GF_MMA_AHEAD;
#endif
    bool ok = true;
    for (int i0 = 0; i0 < nkb && ok; i0 += AHEAD) {
      const int n = min(AHEAD, nkb - i0);
      const int mine = i0 + min(lane, n - 1);
      ok = mbar_wait_lanes(full + mine % STAGES, (uint32_t)(mine / STAGES) & 1u, lane < n, err, 2);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (lane == 0) {
        for (int i = i0; i < i0 + n; ++i) {
          const int s = i % STAGES;
          const uint32_t a = smem_u32(tiles + s * (A_BYTES + B_BYTES));
          const uint64_t ad = umma_desc(a), bd = umma_desc(a + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma(tmem, ad + (uint64_t)(k * UMMA_K * 2 >> 4), bd + (uint64_t)(k * UMMA_K * 2 >> 4),
                 idesc, (i > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty + s);          // the stage is free once these MMAs have read it
        }
      }
      __syncwarp();
    }
    if (lane == 0) {
      if (!ok) gave_up = 1;
      umma_commit(acc_full);               // the accumulator is complete
    }
  } else {
    // epilogue warps: TMEM lanes (warp % 4) * 32 .. + 31
    const int q = warp & 3;
    const int n = n0 + q * 32 + lane;
    pdl_wait();                            // nothing is written before the kernel ahead is done
    // 1 / rms of every token of the tile from the partial sums the product before left behind.
    // The 128 epilogue threads share the tile's live tokens, 2^k threads a token (at most a
    // warp), each taking every 2^k-th partial.  The loads go out now, unguarded (clamped: guarded
    // loads wait in line) and sixteen at a time, and are added up, in a fixed order, only after
    // the wait for the accumulator, so that their latency hides behind the product.
    constexpr int SCALE_BATCH = 16;
    const int live = min(BN, M - m0);
    int tpt = 1;
    while (tpt < 32 && tpt * 2 * live <= 128) tpt *= 2;
    const int e = threadIdx.x - 64, sub = e & (tpt - 1);
    float part[SCALE_BATCH];
    if (ex.in_sumsq) {
      const int tok = e / tpt;                           // this thread's token in the first pass of the loop
      const float* src = ex.in_sumsq + m0 + min(tok, live - 1);
#pragma unroll
      for (int u = 0; u < SCALE_BATCH; ++u)
        part[u] = __ldcg(src + (size_t)min(sub + u * tpt, ex.in_parts - 1) * ex.ss_ld);
    }
    const float* scale = ex.in_sumsq ? scale_s : nullptr;
    const bool ok = mbar_wait(acc_full, 0, err, 3);
    if (!ok) gave_up = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ex.in_sumsq) {
      for (int t0 = 0; t0 < BN; t0 += 128 / tpt) {         // the same trip count for every thread
        const int tok = t0 + e / tpt;
        float sum = 0.f;
        if (tok < live) {
          const float* src = ex.in_sumsq + m0 + tok;
          if (t0 == 0) {
#pragma unroll
            for (int u = 0; u < SCALE_BATCH; ++u)
              sum += sub + u * tpt < ex.in_parts ? part[u] : 0.f;
          }
          for (int p0 = sub + (t0 == 0 ? SCALE_BATCH * tpt : 0); p0 < ex.in_parts;
               p0 += SCALE_BATCH * tpt) {
            float t[SCALE_BATCH];
#pragma unroll
            for (int u = 0; u < SCALE_BATCH; ++u)
              t[u] = __ldcg(src + (size_t)min(p0 + u * tpt, ex.in_parts - 1) * ex.ss_ld);
#pragma unroll
            for (int u = 0; u < SCALE_BATCH; ++u) sum += p0 + u * tpt < ex.in_parts ? t[u] : 0.f;
          }
        }
        for (int o = tpt >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if (sub == 0 && tok < BN) scale_s[tok] = rsqrtf(sum * ex.inv_k + ex.in_eps);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
    }
    if (threadIdx.x == 64) GF_STAMP(5);
    if (ok) {
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
      if (split_k == 1) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (m0 + c >= M) break;
          float v[16], sq[16];
          if (nkb > 0) {
            tmem_ld16(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          }
          epilogue16<EPI, OUT>(v, out, ldo, bias, n, m0 + c, M, N, lane, scale ? scale + c : nullptr,
                               ex, sq);
          if (EPI == EPI_RESID) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float t = warp_sum(sq[j]);
              if (lane == 0) sq_s[q * BN + c + j] = t;
            }
          }
        }
      } else if (CLUSTER && push) {
        // send every row's partial sums to the CTA that owns the row's band
        const int band = band_rows(split_k), row = q * 32 + lane;
        const uint32_t owner = (uint32_t)(row / band), me = cluster_rank();
        const uint32_t bar = dsmem_addr(smem_u32(recv_bar), owner);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (m0 + c >= M) break;
          float v[16];
          if (nkb > 0) {
            tmem_ld16(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            st_async_f4(dsmem_addr(smem_u32(recv + recv_at(c >> 4, (int)me, row % band, j, split_k,
                                                           band)),
                                   owner),
                        v[j], v[j + 1], v[j + 2], v[j + 3], bar);
        }
      } else if (CLUSTER) {
        // park this split's partial tile in shared memory (the ring is drained by now):
        // red[token][RED_LD], a warp's lanes writing neighbouring rows
        float* mine = reinterpret_cast<float*>(tiles) + (q * 32 + lane);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (m0 + c >= M) break;          // the reduction reads live tokens only
          float v[16];
          if (nkb > 0) {
            tmem_ld16(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) mine[(size_t)(c + j) * RED_LD] = v[j];
        }
      } else {
        // park this split's partial tile: workspace[tile][split][row (128)][col (BN)]
        const size_t tile = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
        float* mine = workspace + ((tile * split_k + split) * BM + (q * 32 + lane)) * BN;
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          if (m0 + c >= M) break;
          float v[16];
          if (nkb > 0) {
            tmem_ld16(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            __stcg(reinterpret_cast<float4*>(mine + c + j), make_float4(v[j], v[j + 1], v[j + 2],
                                                                        v[j + 3]));
        }
      }
    }
    if (CLUSTER && push) {
      // this CTA's band, summed over what the peers sent, in rank order
      float* sqs = recv + recv_bytes(BN, split_k) / sizeof(float);
      ReduceBySplit<BN, EPI, OUT>::template run<true>(split_k, 0u, recv, recv_bar, err, bias, out,
                                                      ldo, M, N, n0, m0, scale, ex, sqs);
      if (threadIdx.x == 64) GF_STAMP(6);
    }
    if (EPI == EPI_RESID && split_k == 1) {
      // every epilogue warp arrives, also one whose wait ran out
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int tok = threadIdx.x - 64; tok < BN && ok; tok += 128)
        if (m0 + tok < M)
          ex.out_sumsq[(size_t)blockIdx.x * ex.ss_ld + m0 + tok] =
              (sq_s[tok] + sq_s[BN + tok]) + (sq_s[2 * BN + tok] + sq_s[3 * BN + tok]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (gave_up) {
    // a role left its loop early: copies of this CTA that nobody consumed may still be on their
    // way into its shared memory.  Wait for the last one asked for in each stage (bounded).
    if (threadIdx.x == 0) {
      for (int s = 0; s < STAGES; ++s) {
        int last = -1;
        for (int i = s; i < issued_s; i += STAGES)
          if (i != kSkipped) last = i;
        if (last >= 0) mbar_wait(full + s, (last / STAGES) & 1, nullptr, 0);
      }
    }
    __syncthreads();
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(TMEM_COLS)
                 : "memory");
  }
  if (split_k == 1 || push) {
    if (threadIdx.x == 0) GF_STAMP(push ? 7 : 6);
    return;
  }
  const float* scale = ex.in_sumsq ? scale_s : nullptr;

  if (CLUSTER) {
    // every CTA of the cluster sums a band of rows over all peers, in rank order (the reduction
    // begins with the cluster's barrier)
    pdl_wait();
    const uint32_t red = smem_u32(tiles);
    float* sqs = reinterpret_cast<float*>(tiles) + (size_t)BN * RED_LD;    // behind the parked tile
    ReduceBySplit<BN, EPI, OUT>::template run<false>(split_k, red, nullptr, nullptr, err, bias, out,
                                                     ldo, M, N, n0, m0, scale, ex, sqs);
    if (threadIdx.x == 0) GF_STAMP(6);
    cluster_sync();                                   // nobody leaves while a peer still reads it
    if (threadIdx.x == 0) GF_STAMP(7);
    return;
  }

  // the split that finishes this tile last adds the partials up in split order (the launcher
  // refuses EPI_RESID here: its sums of squares are formed per split)
  __threadfence();
  __syncthreads();
  const unsigned int tile = blockIdx.y * gridDim.x + blockIdx.x;
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&g_tile_done[tile], 1u);
    is_last = done == (unsigned int)split_k - 1;
    if (is_last) g_tile_done[tile] = 0;
  }
  __syncthreads();
  if (!is_last || warp < 2) return;
  __threadfence();
  const int q = warp & 3;
  const int row = q * 32 + lane, n = n0 + row;
  const float* base = workspace + ((size_t)tile * split_k * BM + row) * BN;
#pragma unroll 1
  for (int c = 0; c < BN; c += 16) {
    if (m0 + c >= M) break;
    float v[16], sq[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = 0.f;
    for (int s = 0; s < split_k; ++s) {
      const float* p = base + (size_t)s * BM * BN + c;
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 t = __ldcg(reinterpret_cast<const float4*>(p + j));
        v[j] += t.x;
        v[j + 1] += t.y;
        v[j + 2] += t.z;
        v[j + 3] += t.w;
      }
    }
    epilogue16<EPI, OUT>(v, out, ldo, bias, n, m0 + c, M, N, lane, scale ? scale + c : nullptr, ex,
                         sq);
  }
}

template <int BN, int EPI, typename OUT, bool CLUSTER, bool PUSH = false>
static int launch_mode(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out,
                       int ldo, int M, int N, int K, int split_k, float* workspace, int* err,
                       cudaStream_t st, const GemmExtra& ex) {
  constexpr int STAGES = stages_for(BN);
  const size_t ring = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2);
  // the parked tile of a cluster split, and behind it the squares of an EPI_RESID band (at most
  // 16 row quads x BN tokens)
  const size_t red = CLUSTER ? (size_t)BN * RED_LD * sizeof(float) +
                                   (EPI == EPI_RESID ? (size_t)16 * BN * sizeof(float) : 0)
                             : 0;
  const size_t smem = 1024 + (ring > red ? ring : red) + (2 * STAGES + 2) * sizeof(uint64_t) + 16 +
                      5 * BN * sizeof(float);
  auto k = gemm_tc_kernel<BN, EPI, OUT, CLUSTER, PUSH>;
  static OncePerDevice attrs, np_attrs;              // (of this instantiation of the launcher)
  if (int rc = attrs.run([&] {
        return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      }))
    return rc;
  if (CLUSTER && split_k > 8) {                       // clusters of more than 8 CTAs are opt-in
    if (int rc = np_attrs.run([&] {
          return cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        }))
      return rc;
  }
  dim3 grid((N + BM - 1) / BM, (M + BN - 1) / BN, split_k);
  return launch_kernel_cluster(k, grid, dim3(NTHREADS), smem, st, CLUSTER ? split_k : 1, mw, mx,
                               bias, (OUT*)out, ldo, M, N, K, split_k, workspace, err, ex);
}

template <int BN, int EPI, typename OUT>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out,
                  int ldo, int M, int N, int K, int split_k, float* workspace, int* err,
                  cudaStream_t st, const GemmExtra& ex) {
#ifndef GF_NO_PUSH                                   // (a build to compare the two ways with)
  // (token tiles above 32 have no stages to spare but for very short reductions: not compiled)
  if constexpr (BN <= 32) {
    if (split_k > 1 && !workspace && push_fits<BN, EPI>(K, split_k))
      return launch_mode<BN, EPI, OUT, true, true>(mw, mx, bias, out, ldo, M, N, K, split_k,
                                                   workspace, err, st, ex);
  }
#endif
  if (split_k > 1 && !workspace)
    return launch_mode<BN, EPI, OUT, true>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace,
                                           err, st, ex);
  return launch_mode<BN, EPI, OUT, false>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err,
                                          st, ex);
}

template <int EPI, typename OUT>
static int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const float* bias,
                       void* out, int ldo, int M, int N, int K, int split_k, float* workspace,
                       int* err, cudaStream_t st, const GemmExtra& ex) {
#define GF_CASE(B) \
  case B: return launch<B, EPI, OUT>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err, st, ex)
  switch (bn) {
    GF_CASE(16);
    GF_CASE(32);
    GF_CASE(64);
  }
  if (EPI != EPI_RESID) {       // the residual epilogue serves the token tiles of decode steps only
    switch (bn) {
      GF_CASE(128);
      GF_CASE(256);
    }
  }
#undef GF_CASE
  return -7;
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

#ifdef GF_STAMPS
// Copies the records to `host` (kStampCap * 8 words), returns how many were written, resets.
GF_EXPORT int gf_gemm_bf16_read_stamps(unsigned long long* host) {
  unsigned int n = 0, zero = 0;
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(&n, g_stamp_next, sizeof(n));
  cudaMemcpyFromSymbol(host, g_stamps, sizeof(unsigned long long) * kStampCap * 8);
  cudaMemcpyToSymbol(g_stamp_next, &zero, sizeof(zero));
  return (int)(n < kStampCap ? n : kStampCap);
}
#endif

GF_EXPORT int gf_gemm_bf16_token_tile(int M) {
  return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
}

// fp32 words of workspace that split_k > 1 needs.
GF_EXPORT long long gf_gemm_bf16_workspace_words(int M, int N, int split_k) {
  if (split_k <= 1) return 0;
  const int bn = gf_gemm_bf16_token_tile(M);
  const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
  return tiles * split_k * BM * bn;
}

// out[M, *] = x[M, K] * W[N, K]^T.  epi 0: out[m, n] = acc + bias[n]; epi 2: W rows interleaved
// (gate_i, up_i), out[m, i] = silu(gate) * up, N even; epi 3: out (fp32) = resid + acc + bias with
// out_scaled = bf16(out * gamma[n]) (if given) and out_sumsq[part][m] = the part's share of
// sum_n out^2, parts = gf_gemm_bf16_parts(N, split_k) rows of ss_ld floats; ldo == N, M <= 64,
// cluster mode or no split.  out_f32: fp32 output (epi 0, 3).  ldx, ldo in elements.
// in_sumsq (in_parts rows of ss_ld floats): the accumulator of token m is multiplied by
// rsqrt(sum_p in_sumsq[p][m] / K + in_eps) before bias and epilogue.
// split_k > 1 with a workspace: workspace mode; without: cluster mode (split_k 2, 4, 8 or 12).
// err: a device int that receives a non-zero code if a wait ran out.
// Returns -6 when the shape or alignment cannot be served (the caller uses another product).
GF_EXPORT int gf_gemm_bf16_parts(int N, int split_k) {
  return ((N + BM - 1) / BM) * (split_k < 1 ? 1 : split_k);
}

GF_EXPORT int gf_gemm_bf16_tc_ex(const void* x, int ldx, const void* w, const float* bias,
                                 void* out, int ldo, int M, int N, int K, int epi, int out_f32,
                                 int split_k, void* workspace, int* err, void* stream,
                                 const float* in_sumsq, int in_parts, int ss_ld, float in_eps,
                                 const float* resid, void* out_scaled, const void* gamma,
                                 int gamma_f32, float* out_sumsq) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return -6;
  if (epi == EPI_SILU && ((N & 1) || out_f32)) return -6;
  if (epi != EPI_STORE && epi != EPI_SILU && epi != EPI_RESID) return -6;
  const int bn = gf_gemm_bf16_token_tile(M);
  if (split_k < 1) split_k = 1;
  if (epi == EPI_RESID) {
    if (!out_f32 || !resid || !out_sumsq || ldo != N || bn > 64 || (split_k > 1 && workspace) ||
        ss_ld < M || (out_scaled && !gamma))
      return -6;
  }
  if (in_sumsq && (in_parts <= 0 || ss_ld < M)) return -6;
  const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
  // split_k > 1 without a workspace asks for cluster mode
  if (split_k > 1 && !workspace && split_k != 2 && split_k != 4 && split_k != 8 && split_k != 12)
    return -6;
  if (split_k > 1 && workspace && tiles > kMaxTiles) return -6;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, K, BM) || !make_map(&mx, x, M, K, ldx, bn)) return -6;
  GemmExtra ex = {};
  ex.in_sumsq = in_sumsq;
  ex.in_parts = in_parts;
  ex.ss_ld = ss_ld;
  ex.in_eps = in_eps;
  ex.inv_k = 1.0f / (float)K;
  ex.resid = resid;
  ex.out_scaled = (bf16*)out_scaled;
  ex.gamma = gamma;
  ex.gamma_f32 = gamma_f32;
  ex.out_sumsq = out_sumsq;
  auto st = (cudaStream_t)stream;
  float* ws = (float*)workspace;
  if (epi == EPI_SILU)
    return dispatch_bn<EPI_SILU, bf16>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st,
                                       ex);
  if (epi == EPI_RESID)
    return dispatch_bn<EPI_RESID, float>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st,
                                         ex);
  if (out_f32)
    return dispatch_bn<EPI_STORE, float>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st,
                                         ex);
  return dispatch_bn<EPI_STORE, bf16>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st, ex);
}

GF_EXPORT int gf_gemm_bf16_tc(const void* x, int ldx, const void* w, const float* bias, void* out,
                              int ldo, int M, int N, int K, int epi, int out_f32, int split_k,
                              void* workspace, int* err, void* stream) {
  return gf_gemm_bf16_tc_ex(x, ldx, w, bias, out, ldo, M, N, K, epi, out_f32, split_k, workspace,
                            err, stream, nullptr, 0, 0, 0.f, nullptr, nullptr, nullptr, 0, nullptr);
}
