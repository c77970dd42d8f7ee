// Matrix products of a decode step (at most 32 tokens) with the residual addition and the RMS
// normalisation folded into them, so that a layer needs no separate norm kernels:
//
//   producer  (o_proj, down_proj):   s = residual + x W^T (+ b)            -> fp32, the new residual
//                                    sumsq[part][token] = sum over the part's rows of s^2
//   consumer  (qkv, gate/up, head):  y = norm(s) W^T (+ b)   or   silu(gate) * up
//             where norm(s)[token, k] = bf16(s * gamma[k] * (1 / rms[token])),
//             rms = sqrtf(sum_parts sumsq / K + eps): the formula of the stand-alone norm kernel
//             (csrc/elementwise.cu), which divides by rms where this one multiplies by 1 / rms
//             (one fp32 ulp before the rounding to bf16) and adds the squares in another order.
//
// The consumer does not load its activation operand by TMA: the four epilogue warps read the fp32
// residual rows, normalise them and write the bf16 operand tiles for the CTA's K range into shared
// memory in the 128-byte-swizzled layout the tensor core expects, while the weight tiles stream in
// by TMA.  Everything else is the tcgen05 kernel of csrc/gemm_bf16.cu at small token tiles: weights
// are the A operand (128 rows = TMEM lanes), tokens the columns; split-K by thread-block clusters
// with the reduction through distributed shared memory; weights prefetched before
// griddepcontrol.wait; bounded mbarrier waits.
//
// The reference has separate add, RMSNorm and cuBLASLt launches for all of this
// (ginfer/core/layer/transformer/encoder.cc:33-39).
#include "tc_common.cuh"

namespace gf {

constexpr int NTHREADS = 192;
constexpr int MAX_STAGES = 10;      // the launcher takes as many as fit beside the operand tiles
constexpr int EPI_STORE = 0, EPI_SILU = 2, EPI_RESID = 3;
constexpr int kMaxParts = 1024;

struct FuseArgs {
  // producer
  const float* resid_in;     // [M, N] fp32
  float* sumsq_out;          // [parts, ss_ld]
  // consumer
  const float* b_resid;      // [M, K] fp32: the operand before normalisation
  const float* b_sumsq;      // [b_parts, ss_ld]
  const void* gamma;         // [K]
  int gamma_f32;
  int b_parts;
  int ss_ld;
  float eps;
};

template <typename OUT> __device__ __forceinline__ void put(OUT* p, float v);
template <> __device__ __forceinline__ void put<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ void put<float>(float* p, float v) { *p = v; }

__device__ __forceinline__ float silu_mul(float g, float u) {
  const float gg = __bfloat162float(__float2bfloat16_rn(g));
  const float uu = __bfloat162float(__float2bfloat16_rn(u));
  return gg * (1.0f / (1.0f + expf(-gg))) * uu;
}

template <int BN, int EPI, typename OUT, bool NORMB>
__global__ void __launch_bounds__(NTHREADS)
gemm_fused_kernel(const __grid_constant__ CUtensorMap tmap_w,
                  const __grid_constant__ CUtensorMap tmap_x, const float* __restrict__ bias,
                  OUT* __restrict__ out, int ldo, int M, int N, int K, int split_k,
                  const int STAGES, const FuseArgs fa, int* __restrict__ err) {
  static_assert(BN == 16 || BN == 32, "token tiles of 16 or 32");
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + (NORMB ? 0 : B_BYTES);
  constexpr uint32_t TMEM_COLS = 32;
  constexpr uint32_t RED_BYTES = BM * (BN + 4) * 4;          // parked partial tile
  constexpr uint32_t SQ_BYTES = BM * BN * 4;                  // squares for the row sums
  const uint32_t REGION0 = STAGES * STAGE_BYTES > RED_BYTES + SQ_BYTES
                               ? STAGES * STAGE_BYTES : RED_BYTES + SQ_BYTES;
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * BM, split = blockIdx.z;
  const int nkb_all = (K + BK - 1) / BK;
  const int per = (nkb_all + split_k - 1) / split_k;
  const int kb0 = split * per, kb1 = min(nkb_all, kb0 + per);
  const int nkb = max(0, kb1 - kb0);

  unsigned char* bres = tiles + REGION0;                      // NORMB: [per][BN][64] bf16
  uint64_t* full = (uint64_t*)(bres + (NORMB ? (size_t)per * B_BYTES : 0));
  uint64_t* empty = full + STAGES;
  uint64_t* acc_full = empty + STAGES;
  uint64_t* b_ready = acc_full + 1;
  uint32_t* tmem_slot = (uint32_t*)(b_ready + 1);
  float* rms_s = (float*)(tmem_slot + 2);                     // [BN]

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(b_ready, 128);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
    if (!NORMB) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
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
      // weights first (they do not depend on the kernel before), then the activations
      const int pre = nkb < STAGES ? nkb : STAGES;
      for (int i = 0; i < pre; ++i) {
        mbar_expect_tx(full + i, STAGE_BYTES);
        tma_load_2d(tiles + i * STAGE_BYTES, &tmap_w, full + i, (kb0 + i) * BK, n0);
      }
      pdl_wait();
      if (!NORMB)
        for (int i = 0; i < pre; ++i)
          tma_load_2d(tiles + i * STAGE_BYTES + A_BYTES, &tmap_x, full + i, (kb0 + i) * BK, 0);
      for (int i = pre; i < nkb; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(empty + s, ((i / STAGES) & 1) ^ 1, err, 1)) break;
        mbar_expect_tx(full + s, STAGE_BYTES);
        unsigned char* a = tiles + s * STAGE_BYTES;
        tma_load_2d(a, &tmap_w, full + s, (kb0 + i) * BK, n0);
        if (!NORMB) tma_load_2d(a + A_BYTES, &tmap_x, full + s, (kb0 + i) * BK, 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                 ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
      bool ok = true;
      if (NORMB) ok = mbar_wait(b_ready, 0, err, 4);          // the normalised operand is written
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % STAGES;
        ok = mbar_wait(full + s, (i / STAGES) & 1, err, 2);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a = smem_u32(tiles + s * STAGE_BYTES);
        const uint32_t b = NORMB ? smem_u32(bres + (size_t)i * B_BYTES) : a + A_BYTES;
        const uint64_t ad = umma_desc(a), bd = umma_desc(b);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma(tmem, ad + (uint64_t)(k * UMMA_K * 2 >> 4), bd + (uint64_t)(k * UMMA_K * 2 >> 4),
               idesc, (i > 0 || k > 0) ? 1u : 0u);
        umma_commit(empty + s);
      }
      umma_commit(acc_full);
    }
  } else {
    const int q = warp & 3;
    const int e = threadIdx.x - 64;                           // 0 .. 127
    pdl_wait();
    if (NORMB) {
      // 1. rms of every token from the producer's partial sums: 128 / BN threads a token, each
      //    over every (128 / BN)-th part, then a fixed shuffle tree (the order of the additions
      //    depends on nothing but the number of parts)
      {
        constexpr int TPT = 128 / BN;                          // threads per token: 8 or 4
        const int m = e / TPT, sub = e % TPT;
        float ss = 0.f;
        if (m < M)
          for (int p = sub; p < fa.b_parts; p += TPT)
            ss += __ldg(fa.b_sumsq + (size_t)p * fa.ss_ld + m);
#pragma unroll
        for (int o = TPT / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (sub == 0) rms_s[m] = 1.0f / sqrtf(ss / (float)K + fa.eps);   // one division a token
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");          // the four epilogue warps only
      // 2. this CTA's K range of the operand: bf16(s * gamma / rms), 8 channels (16 bytes) a time.
      //    The loads of four chunks are issued together and without branches (addresses are
      //    clamped, results of clamped loads dropped); rows past the last token are zero.
      //    Thread e owns channel group e & 7 of the rows e >> 3, + 16, + 32, ... of the list of
      //    (k block, token) pairs; the pair is advanced without divisions.
      const int ch = e & 7;
      const int pairs = nkb * M;
      const int step_k = 16 / M, step_m = 16 % M;
      int j = e >> 3, kbl = j / M, m = j % M;
      const int k_last = K - 8;                                 // K is a multiple of 8
      while (j < pairs) {
        float4 s0[4], s1[4], g0[4], g1[4];
        int kbl_u[4], m_u[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          kbl_u[u] = kbl, m_u[u] = m;
          const int kc = min(kbl, nkb - 1);
          const int k = min((kb0 + kc) * BK + ch * 8, k_last);
          const float4* sp = reinterpret_cast<const float4*>(fa.b_resid + (size_t)m * K + k);
          s0[u] = __ldg(sp);
          s1[u] = __ldg(sp + 1);
          if (fa.gamma_f32) {
            g0[u] = __ldg(reinterpret_cast<const float4*>((const float*)fa.gamma + k));
            g1[u] = __ldg(reinterpret_cast<const float4*>((const float*)fa.gamma + k + 4));
          } else {
            const uint4 gr = __ldg(reinterpret_cast<const uint4*>((const bf16*)fa.gamma + k));
            const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
            const float2 a0 = __bfloat1622float2(gp[0]), a1 = __bfloat1622float2(gp[1]);
            const float2 a2 = __bfloat1622float2(gp[2]), a3 = __bfloat1622float2(gp[3]);
            g0[u] = make_float4(a0.x, a0.y, a1.x, a1.y);
            g1[u] = make_float4(a2.x, a2.y, a3.x, a3.y);
          }
          kbl += step_k, m += step_m;
          if (m >= M) m -= M, ++kbl;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (j + 16 * u < pairs) {
            const int mm = m_u[u];
            const int k = (kb0 + kbl_u[u]) * BK + ch * 8;
            uint4 w = make_uint4(0u, 0u, 0u, 0u);
            if (k < K) {
              // multiplied by 1/rms: at four warps a CTA the eight IEEE divisions a chunk that
              // the stand-alone norm kernel makes cost microseconds here (the result differs
              // from that kernel's by at most one fp32 ulp before the rounding to bf16)
              const float r = rms_s[mm];
              __nv_bfloat162 t0 = __floats2bfloat162_rn(s0[u].x * g0[u].x * r, s0[u].y * g0[u].y * r);
              __nv_bfloat162 t1 = __floats2bfloat162_rn(s0[u].z * g0[u].z * r, s0[u].w * g0[u].w * r);
              __nv_bfloat162 t2 = __floats2bfloat162_rn(s1[u].x * g1[u].x * r, s1[u].y * g1[u].y * r);
              __nv_bfloat162 t3 = __floats2bfloat162_rn(s1[u].z * g1[u].z * r, s1[u].w * g1[u].w * r);
              w = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1),
                             *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
            }
            *reinterpret_cast<uint4*>(bres + (size_t)kbl_u[u] * B_BYTES + mm * 128 +
                                      ((ch ^ (mm & 7)) << 4)) = w;
          }
        }
        j += 64;
      }
      for (int kb = e >> 3; kb < nkb; kb += 16)
        for (int mm = M; mm < BN; ++mm)
          *reinterpret_cast<uint4*>(bres + (size_t)kb * B_BYTES + mm * 128 +
                                    ((ch ^ (mm & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(b_ready);
    }
    const bool ok = mbar_wait(acc_full, 0, err, 3);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
    const int rowl = q * 32 + lane, n = n0 + rowl;
    if (ok && split_k > 1) {
      // park this split's partial tile in shared memory (the ring is drained by now)
      float* mine = reinterpret_cast<float*>(tiles) + (size_t)rowl * (BN + 4);
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        if (nkb > 0) {
          tmem_ld16(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 16; j += 4)
          *reinterpret_cast<float4*>(mine + c + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
      }
    } else if (ok) {
      // no split: the epilogue straight from tensor memory
      float* sq = reinterpret_cast<float*>(tiles + RED_BYTES);   // [128][BN]
#pragma unroll
      for (int c = 0; c < BN; c += 16) {
        float v[16];
        tmem_ld16(taddr + c, v);
        if (EPI == EPI_SILU) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
            if ((j & 1) == (lane & 1) && (n | 1) < N && c + j < M)
              put<OUT>(out + (size_t)(c + j) * ldo + (n >> 1),
                       (lane & 1) ? silu_mul(other, v[j]) : silu_mul(v[j], other));
          }
        } else {
          const float b = (bias && n < N) ? bias[n] : 0.f;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float s = v[j] + b;
            const bool in = n < N && c + j < M;
            if (EPI == EPI_RESID) {
              if (in) s += fa.resid_in[(size_t)(c + j) * N + n];
              sq[rowl * BN + c + j] = in ? s * s : 0.f;
            }
            if (in) put<OUT>(out + (size_t)(c + j) * ldo + n, s);
          }
        }
      }
    }
    if (EPI == EPI_RESID && split_k == 1) {
      // every epilogue thread comes here, whether its wait ran out or not
      asm volatile("bar.sync 1, 128;" ::: "memory");
      const float* sq = reinterpret_cast<const float*>(tiles + RED_BYTES);
      if (ok)
        for (int m = e; m < BN; m += 128) {
          float ss = 0.f;
          for (int r = 0; r < BM; ++r) ss += sq[r * BN + m];
          fa.sumsq_out[(size_t)blockIdx.x * fa.ss_ld + m] = ss;
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

  // every CTA of the cluster sums a band of rows over all peers, in rank order
  pdl_wait();
  cluster_sync();
  const int rank = (int)cluster_rank();
  const int band = BM / split_k;                      // split_k is 2, 4 or 8
  constexpr int QUADS = BN / 4;
  const uint32_t red = smem_u32(tiles);
  float* sq = reinterpret_cast<float*>(tiles + RED_BYTES);      // [band][BN]
  if (EPI == EPI_SILU) {
    const int pairs = band / 2;
    for (int u = threadIdx.x; u < pairs * QUADS; u += NTHREADS) {
      const int row = rank * band + 2 * (u % pairs), c = (u / pairs) * 4;
      if (c >= M || n0 + row + 1 >= N) continue;
      float4 g = make_float4(0.f, 0.f, 0.f, 0.f), up = g;
#pragma unroll 8
      for (int p = 0; p < split_k; ++p) {
        const float4 a = ld_dsmem_f4(red + (uint32_t)((row * (BN + 4) + c) * 4), p);
        const float4 b = ld_dsmem_f4(red + (uint32_t)(((row + 1) * (BN + 4) + c) * 4), p);
        g.x += a.x, g.y += a.y, g.z += a.z, g.w += a.w;
        up.x += b.x, up.y += b.y, up.z += b.z, up.w += b.w;
      }
      const float gv[4] = {g.x, g.y, g.z, g.w}, uv[4] = {up.x, up.y, up.z, up.w};
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (c + j < M)
          put<OUT>(out + (size_t)(c + j) * ldo + ((n0 + row) >> 1), silu_mul(gv[j], uv[j]));
    }
  } else {
    if (EPI == EPI_RESID) {
      for (int i = threadIdx.x; i < band * BN; i += NTHREADS) sq[i] = 0.f;
      __syncthreads();
    }
    for (int u = threadIdx.x; u < band * QUADS; u += NTHREADS) {
      const int rl = u % band, row = rank * band + rl, c = (u / band) * 4;
      const int n = n0 + row;
      if (c >= M || n >= N) continue;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
      for (int p = 0; p < split_k; ++p) {
        const float4 t = ld_dsmem_f4(red + (uint32_t)((row * (BN + 4) + c) * 4), p);
        v.x += t.x, v.y += t.y, v.z += t.z, v.w += t.w;
      }
      const float b = bias ? bias[n] : 0.f;
      float vv[4] = {v.x + b, v.y + b, v.z + b, v.w + b};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (c + j >= M) continue;
        if (EPI == EPI_RESID) {
          vv[j] += fa.resid_in[(size_t)(c + j) * N + n];
          sq[rl * BN + c + j] = vv[j] * vv[j];
        }
        put<OUT>(out + (size_t)(c + j) * ldo + n, vv[j]);
      }
    }
    if (EPI == EPI_RESID) {
      __syncthreads();
      for (int m = threadIdx.x; m < BN; m += NTHREADS) {
        float ss = 0.f;
        for (int r = 0; r < band; ++r) ss += sq[r * BN + m];
        fa.sumsq_out[((size_t)blockIdx.x * split_k + rank) * fa.ss_ld + m] = ss;
      }
    }
  }
  cluster_sync();                                     // nobody leaves while a peer still reads it
}

template <int BN, int EPI, typename OUT, bool NORMB>
static int launch_fused(const CUtensorMap& mw, const CUtensorMap& mx, const float* bias, void* out,
                        int ldo, int M, int N, int K, int split_k, const FuseArgs& fa, int* err,
                        cudaStream_t st) {
  const int nkb_all = (K + BK - 1) / BK, per = (nkb_all + split_k - 1) / split_k;
  constexpr size_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr size_t STAGE = A_BYTES + (NORMB ? 0 : B_BYTES);
  constexpr size_t RED = BM * (BN + 4) * 4 + BM * BN * 4;
  const size_t bres = NORMB ? (size_t)per * B_BYTES : 0;
  const size_t fixed = 1024 + bres + (2 * MAX_STAGES + 2) * sizeof(uint64_t) + 8 + BN * 4 + 16;
  int stages = per < MAX_STAGES ? per : MAX_STAGES;
  if (stages < 2) stages = 2;
  // one wave: the deepest ring that fits (weights stream in while the operand is normalised);
  // several waves: two CTAs to an SM, so that one streams while the other starts up
  const size_t ctas = (size_t)((N + BM - 1) / BM) * split_k;
  const size_t room = ctas > 148 ? 112 * 1024 : 200 * 1024;
  while (stages > 2 && fixed + stages * STAGE > room) --stages;
  const size_t region0 = stages * STAGE > RED ? stages * STAGE : RED;
  const size_t smem = fixed + region0;
  if (smem > 200 * 1024) return -6;
  auto k = gemm_fused_kernel<BN, EPI, OUT, NORMB>;
  static size_t attr = 0;
  if (smem > attr) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr = smem;
  }
  dim3 grid((N + BM - 1) / BM, 1, split_k);
  return launch_kernel_cluster(k, grid, dim3(NTHREADS), smem, st, split_k, mw, mx, bias, (OUT*)out,
                               ldo, M, N, K, split_k, stages, fa, err);
}

template <int BN>
static int dispatch(int mode, const CUtensorMap& mw, const CUtensorMap& mx, const float* bias,
                    void* out, int ldo, int M, int N, int K, int split_k, const FuseArgs& fa,
                    int out_f32, int* err, cudaStream_t st) {
  // mode: 0 normed -> bf16/fp32 (+bias), 1 normed -> silu(gate) * up, 2 plain -> residual + stats
  if (mode == 0 && out_f32)
    return launch_fused<BN, EPI_STORE, float, true>(mw, mx, bias, out, ldo, M, N, K, split_k, fa,
                                                    err, st);
  if (mode == 0)
    return launch_fused<BN, EPI_STORE, bf16, true>(mw, mx, bias, out, ldo, M, N, K, split_k, fa,
                                                   err, st);
  if (mode == 1)
    return launch_fused<BN, EPI_SILU, bf16, true>(mw, mx, bias, out, ldo, M, N, K, split_k, fa, err,
                                                  st);
  return launch_fused<BN, EPI_RESID, float, false>(mw, mx, bias, out, ldo, M, N, K, split_k, fa, err,
                                                   st);
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

// Producer: resid_out[M, N] (fp32) = resid_in + x[M, K] W[N, K]^T (+ bias); sumsq_out[parts, ss_ld]
// with parts = ceil(N / 128) * split_k receives each part's sum of squares per token.
// M <= 32; split_k 1, 2, 4 or 8.  Returns -6 for what it cannot serve.
GF_EXPORT int gf_gemm_resid(const void* x, int ldx, const void* w, const float* bias,
                            const float* resid_in, float* resid_out, float* sumsq_out, int ss_ld,
                            int M, int N, int K, int split_k, int* err, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K <= 0 || K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return -6;
  if (split_k != 1 && split_k != 2 && split_k != 4 && split_k != 8) return -6;
  const int bn = M <= 16 ? 16 : 32;
  if (ss_ld < bn || (long long)((N + BM - 1) / BM) * split_k > kMaxParts) return -6;
  CUtensorMap mw, mx;
  if (!make_map(&mw, w, N, K, K, BM) || !make_map(&mx, x, M, K, ldx, bn)) return -6;
  FuseArgs fa = {};
  fa.resid_in = resid_in;
  fa.sumsq_out = sumsq_out;
  fa.ss_ld = ss_ld;
  auto st = (cudaStream_t)stream;
  if (bn == 16) return dispatch<16>(2, mw, mx, bias, resid_out, N, M, N, K, split_k, fa, 1, err, st);
  return dispatch<32>(2, mw, mx, bias, resid_out, N, M, N, K, split_k, fa, 1, err, st);
}

// Consumer: out = norm(resid)[M, K] W[N, K]^T (+ bias), or with gated != 0 (W rows interleaved
// gate_i, up_i) out[M, N / 2] = silu(gate) * up.  norm(resid) = bf16(resid * gamma / rms) with
// rms from the producer's sumsq[b_parts, ss_ld].  M <= 32; K % 8 == 0; the CTA's share of the
// operand must fit its shared memory (K / split_k up to about 2048 at 16 tokens).
GF_EXPORT int gf_gemm_normed(const float* resid, const float* sumsq, int b_parts, int ss_ld,
                             const void* gamma, int gamma_f32, float eps, const void* w,
                             const float* bias, void* out, int ldo, int M, int N, int K, int gated,
                             int out_f32, int split_k, int* err, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 32 || K <= 0 || K % 8 || ((uintptr_t)resid & 15) || ((uintptr_t)w & 15) ||
      ((uintptr_t)gamma & 15))
    return -6;
  if (split_k != 1 && split_k != 2 && split_k != 4 && split_k != 8) return -6;
  if (gated && ((N & 1) || out_f32)) return -6;
  const int bn = M <= 16 ? 16 : 32;
  if (ss_ld < bn || b_parts <= 0) return -6;
  CUtensorMap mw;
  if (!make_map(&mw, w, N, K, K, BM)) return -6;
  FuseArgs fa = {};
  fa.b_resid = resid;
  fa.b_sumsq = sumsq;
  fa.gamma = gamma;
  fa.gamma_f32 = gamma_f32;
  fa.b_parts = b_parts;
  fa.ss_ld = ss_ld;
  fa.eps = eps;
  auto st = (cudaStream_t)stream;
  if (bn == 16)
    return dispatch<16>(gated ? 1 : 0, mw, mw, bias, out, ldo, M, N, K, split_k, fa, out_f32, err, st);
  return dispatch<32>(gated ? 1 : 0, mw, mw, bias, out, ldo, M, N, K, split_k, fa, out_f32, err, st);
}
