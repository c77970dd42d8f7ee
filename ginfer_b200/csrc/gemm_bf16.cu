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
// Products whose tiles alone would leave most SMs idle (the small-N products of a decode step) split
// the K range, deterministically, in one of two ways.  Cluster mode (split_k 2, 4 or 8): the splits
// of a tile form a thread-block cluster, park their fp32 partial tiles in their own shared memory,
// and after a cluster barrier each CTA sums a band of rows over all peers through distributed
// shared memory, in rank order, and runs the epilogue for it.  Workspace mode (any split_k): the
// partials go to global memory and the split that finishes a tile last (counted with an atomic it
// resets) sums them in split order.
//
// The reference calls cuBLASLt for every product (ginfer/core/op/kernels/cuda/gemm_kernel/
// gemm_kernel.cu:93-156, bias in the epilogue :112-121, fp32 compute :100) and has a separate
// SwiGLU kernel (swiglu_kernel.cu:6-31).
//
// Every wait on an mbarrier is bounded: after kSpinLimit polls the waiter records an error code in
// *err and leaves its loop; all roles then meet at the final barrier and tensor memory is freed.
#include "tc_common.cuh"

namespace gf {

constexpr int NTHREADS = 192;
constexpr int EPI_STORE = 0, EPI_SILU = 2;
constexpr int kMaxTiles = 1 << 16;
__device__ unsigned int g_tile_done[kMaxTiles];

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

// Epilogue of 16 accumulator columns (tokens m_base .. m_base + 15) of W row n for one thread.
template <int EPI, typename OUT>
__device__ __forceinline__ void epilogue16(float (&v)[16], OUT* __restrict__ out, int ldo,
                                           const float* __restrict__ bias, int n, int m_base,
                                           int M, int N, int lane) {
  if (EPI == EPI_STORE) {
    const float b = (bias && n < N) ? bias[n] : 0.f;
    if (n < N) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (m_base + j < M) store_out<OUT>(out + (size_t)(m_base + j) * ldo + n, v[j] + b);
    }
  } else {
    // rows come in pairs (gate, up) on adjacent lanes; each lane finishes every other token
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float mine = __bfloat162float(__float2bfloat16_rn(v[j]));
      const float other = __shfl_xor_sync(0xffffffffu, mine, 1);
      if ((j & 1) == (lane & 1)) {
        const float g = (lane & 1) ? other : mine, u = (lane & 1) ? mine : other;
        const int pair = n >> 1;
        if ((n | 1) < N && m_base + j < M)
          store_out<OUT>(out + (size_t)(m_base + j) * ldo + pair,
                         g * (1.0f / (1.0f + expf(-g))) * u);
      }
    }
  }
}

// Cluster split-K: every CTA of the cluster sums a band of the tile's rows over all SPLIT peers'
// parked partial tiles, read through distributed shared memory.  The peers' loads are issued
// together and the additions stay in rank order.
template <int BN, int EPI, typename OUT, int SPLIT>
__device__ __forceinline__ void cluster_reduce(uint32_t red, const float* __restrict__ bias,
                                               OUT* __restrict__ out, int ldo, int M, int N,
                                               int n0, int m0) {
  const int rank = (int)cluster_rank();
  constexpr int band = ((BM + SPLIT - 1) / SPLIT + 1) & ~1;   // rows a CTA adds up (even: row pairs)
  constexpr int QUADS = BN / 4;                       // a unit of work: one row (pair), 4 tokens
  if (EPI == EPI_STORE) {
    for (int u = threadIdx.x; u < band * QUADS; u += NTHREADS) {
      const int row = rank * band + u % band, c = (u / band) * 4;
      const int n = n0 + row;
      if (row >= BM || m0 + c >= M || n >= N) continue;
      float4 t[SPLIT];
#pragma unroll
      for (int p = 0; p < SPLIT; ++p)
        t[p] = ld_dsmem_f4(red + (uint32_t)((row * (BN + 4) + c) * 4), p);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int p = 0; p < SPLIT; ++p) v.x += t[p].x, v.y += t[p].y, v.z += t[p].z, v.w += t[p].w;
      const float b = bias ? bias[n] : 0.f;
      const float vv[4] = {v.x + b, v.y + b, v.z + b, v.w + b};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (m0 + c + j < M) store_out<OUT>(out + (size_t)(m0 + c + j) * ldo + n, vv[j]);
    }
  } else {
    constexpr int pairs = band / 2;
    for (int u = threadIdx.x; u < pairs * QUADS; u += NTHREADS) {
      const int row = rank * band + 2 * (u % pairs), c = (u / pairs) * 4;
      const int pair = (n0 + row) >> 1;
      if (row >= BM || m0 + c >= M || n0 + row + 1 >= N) continue;
      float4 ta[SPLIT], tb[SPLIT];
#pragma unroll
      for (int p = 0; p < SPLIT; ++p) {
        ta[p] = ld_dsmem_f4(red + (uint32_t)((row * (BN + 4) + c) * 4), p);
        tb[p] = ld_dsmem_f4(red + (uint32_t)(((row + 1) * (BN + 4) + c) * 4), p);
      }
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f), up = g;
#pragma unroll
      for (int p = 0; p < SPLIT; ++p) {
        g.x += ta[p].x, g.y += ta[p].y, g.z += ta[p].z, g.w += ta[p].w;
        up.x += tb[p].x, up.y += tb[p].y, up.z += tb[p].z, up.w += tb[p].w;
      }
      const float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gg = __bfloat162float(__float2bfloat16_rn(gv[j]));
        const float uu = __bfloat162float(__float2bfloat16_rn(uv[j]));
        if (m0 + c + j < M)
          store_out<OUT>(out + (size_t)(m0 + c + j) * ldo + pair,
                         gg * (1.0f / (1.0f + expf(-gg))) * uu);
      }
    }
  }
}

template <int BN, int EPI, typename OUT, bool CLUSTER>
__global__ void __launch_bounds__(NTHREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
               const float* __restrict__ bias, OUT* __restrict__ out, int ldo, int M, int N, int K,
               int split_k, float* __restrict__ workspace, int* __restrict__ err) {
  constexpr int STAGES = stages_for(BN);
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  uint64_t* full = (uint64_t*)(tiles + STAGES * (A_BYTES + B_BYTES));
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(acc_full + 1);
  __shared__ bool is_last;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, m0 = blockIdx.y * BN, split = blockIdx.z;
  const int nkb_all = (K + BK - 1) / BK;
  const int per = (nkb_all + split_k - 1) / split_k;
  const int kb0 = split * per, kb1 = min(nkb_all, kb0 + per);
  const int nkb = max(0, kb1 - kb0);

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
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

  if (warp == 0) {
    if (lane == 0) {
      // Weights do not depend on the kernel before this one: fill the ring with them first, then
      // wait for that kernel and add the activations to the same stages.
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full + i, A_BYTES + B_BYTES);
        tma_load_2d(tiles + i * (A_BYTES + B_BYTES), &tmap_w, full + i, (kb0 + i) * BK, n0);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i)
        tma_load_2d(tiles + i * (A_BYTES + B_BYTES) + A_BYTES, &tmap_x, full + i, (kb0 + i) * BK,
                    m0);
      for (int i = pre; i < nkb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(empty + s, ((i / STAGES) & 1) ^ 1, err, 1)) break;
        mbar_expect_tx(full + s, A_BYTES + B_BYTES);
        unsigned char* a = tiles + s * (A_BYTES + B_BYTES);
        tma_load_2d(a, &tmap_w, full + s, (kb0 + i) * BK, n0);
        tma_load_2d(a + A_BYTES, &tmap_x, full + s, (kb0 + i) * BK, m0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BN);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(full + s, (i / STAGES) & 1, err, 2);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_u32(tiles + s * (A_BYTES + B_BYTES));
        const uint64_t ad = umma_desc(a), bd = umma_desc(a + A_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma(tmem, ad + (uint64_t)(k * UMMA_K * 2 >> 4), bd + (uint64_t)(k * UMMA_K * 2 >> 4),
               idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty + s);            // the stage is free once these MMAs have read it
      }
      umma_commit(acc_full);               // the accumulator is complete
    }
  } else {
    // epilogue warps: TMEM lanes (warp % 4) * 32 .. + 31
    const int q = warp & 3;
    const int n = n0 + q * 32 + lane;
    pdl_wait();                            // nothing is written before the kernel ahead is done
    const bool ok = mbar_wait(acc_full, 0, err, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
      if (split_k == 1) {
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
          epilogue16<EPI, OUT>(v, out, ldo, bias, n, m0 + c, M, N, lane);
        }
      } else if (CLUSTER) {
        // park this split's partial tile in shared memory (the ring is drained by now):
        // red[row (128)][RED_LD], rows padded so that float4 stores do not collide
        float* mine = reinterpret_cast<float*>(tiles) + (size_t)(q * 32 + lane) * (BN + 4);
#pragma unroll 1
        for (int c = 0; c < BN; c += 16) {
          float v[16];
          if (nkb > 0 && m0 + c < M) {
            tmem_ld16(taddr + c, v);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<float4*>(mine + c + j) = make_float4(v[j], v[j + 1], v[j + 2],
                                                                    v[j + 3]);
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
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(TMEM_COLS)
                 : "memory");
  }
  if (split_k == 1) return;

  if (CLUSTER) {
    // every CTA of the cluster sums a band of rows over all peers, in rank order
    pdl_wait();
    cluster_sync();
    const uint32_t red = smem_u32(tiles);
    if (split_k == 2)
      cluster_reduce<BN, EPI, OUT, 2>(red, bias, out, ldo, M, N, n0, m0);
    else if (split_k == 4)
      cluster_reduce<BN, EPI, OUT, 4>(red, bias, out, ldo, M, N, n0, m0);
    else if (split_k == 8)
      cluster_reduce<BN, EPI, OUT, 8>(red, bias, out, ldo, M, N, n0, m0);
    else
      cluster_reduce<BN, EPI, OUT, 12>(red, bias, out, ldo, M, N, n0, m0);
    cluster_sync();                                   // nobody leaves while a peer still reads it
    return;
  }

  // the split that finishes this tile last adds the partials up in split order
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
    float v[16];
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
    epilogue16<EPI, OUT>(v, out, ldo, bias, n, m0 + c, M, N, lane);
  }
}

template <int BN, int EPI, typename OUT, bool CLUSTER>
static int launch_mode(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out,
                       int ldo, int M, int N, int K, int split_k, float* workspace, int* err,
                       cudaStream_t st) {
  constexpr int STAGES = stages_for(BN);
  const size_t ring = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2);
  const size_t red = CLUSTER ? (size_t)BM * (BN + 4) * sizeof(float) : 0;
  const size_t smem = 1024 + (ring > red ? ring : red) + (2 * STAGES + 1) * sizeof(uint64_t) + 16;
  auto k = gemm_tc_kernel<BN, EPI, OUT, CLUSTER>;
  static bool done = false;
  if (!done) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    done = true;
  }
  if (CLUSTER && split_k > 8) {                       // clusters of more than 8 CTAs are opt-in
    static bool np_done = false;
    if (!np_done) {
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) return (int)e;
      np_done = true;
    }
  }
  dim3 grid((N + BM - 1) / BM, (M + BN - 1) / BN, split_k);
  return launch_kernel_cluster(k, grid, dim3(NTHREADS), smem, st, CLUSTER ? split_k : 1, mw, mx,
                               bias, (OUT*)out, ldo, M, N, K, split_k, workspace, err);
}

template <int BN, int EPI, typename OUT>
static int launch(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out,
                  int ldo, int M, int N, int K, int split_k, float* workspace, int* err,
                  cudaStream_t st) {
  if (split_k > 1 && !workspace)
    return launch_mode<BN, EPI, OUT, true>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace,
                                           err, st);
  return launch_mode<BN, EPI, OUT, false>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err,
                                          st);
}

template <int EPI, typename OUT>
static int dispatch_bn(int bn, const CUtensorMap& mw, const CUtensorMap& mx, const float* bias,
                       void* out, int ldo, int M, int N, int K, int split_k, float* workspace,
                       int* err, cudaStream_t st) {
  switch (bn) {
    case 16: return launch<16, EPI, OUT>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err, st);
    case 32: return launch<32, EPI, OUT>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err, st);
    case 64: return launch<64, EPI, OUT>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err, st);
    case 128: return launch<128, EPI, OUT>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err, st);
    case 256: return launch<256, EPI, OUT>(mw, mx, bias, out, ldo, M, N, K, split_k, workspace, err, st);
  }
  return -7;
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

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
// (gate_i, up_i), out[m, i] = silu(gate) * up, N even.  out_f32: fp32 output (epi 0 only).
// ldx, ldo in elements.  split_k > 1 with a workspace: workspace mode; without: cluster mode
// (split_k 2, 4 or 8).  err: a device int that receives a non-zero code if a wait ran out.
// Returns -6 when the shape or alignment cannot be served (the caller uses another product).
GF_EXPORT int gf_gemm_bf16_tc(const void* x, int ldx, const void* w, const float* bias, void* out,
                              int ldo, int M, int N, int K, int epi, int out_f32, int split_k,
                              void* workspace, int* err, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return -6;
  if (epi == EPI_SILU && ((N & 1) || out_f32)) return -6;
  if (epi != EPI_STORE && epi != EPI_SILU) return -6;
  const int bn = gf_gemm_bf16_token_tile(M);
  if (split_k < 1) split_k = 1;
  const long long tiles = (long long)((N + BM - 1) / BM) * ((M + bn - 1) / bn);
  // split_k > 1 without a workspace asks for cluster mode
  if (split_k > 1 && !workspace && split_k != 2 && split_k != 4 && split_k != 8 && split_k != 12)
    return -6;
  if (split_k > 1 && workspace && tiles > kMaxTiles) return -6;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, K, BM) || !make_map(&mx, x, M, K, ldx, bn)) return -6;
  auto st = (cudaStream_t)stream;
  float* ws = (float*)workspace;
  if (epi == EPI_SILU)
    return dispatch_bn<EPI_SILU, bf16>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st);
  if (out_f32)
    return dispatch_bn<EPI_STORE, float>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st);
  return dispatch_bn<EPI_STORE, bf16>(bn, mw, mx, bias, out, ldo, M, N, K, split_k, ws, err, st);
}
