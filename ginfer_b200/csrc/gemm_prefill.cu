// y[M, N] = x[M, K] @ W[N, K]^T for many tokens (prompt portions): a persistent tcgen05 kernel.
//
// Tiles of 128 tokens x 256 weight rows: the tokens are the 128 rows of the MMA (= TMEM lanes),
// the weight rows its 256 columns, so that a thread of the epilogue owns one token and writes
// runs of neighbouring output channels with 16-byte stores, and a gate finds its up value in the
// next column (weights interleaved gate_0, up_0, gate_1, ...: SiLU*mul is fused, and only the
// product is written: the round trip of gate and up through memory, 110 MB a layer at 2,048
// tokens of the 1.5B shape, goes away).  A third epilogue serves the joined q/k/v product: a
// thread holds whole heads of its token, so it adds the bias, rotates q and k by the token's
// angles and writes k and v into the token's slot of the paged cache as well as into `out` (no
// rotation kernel reads and rewrites q/k/v behind the product); it reads the table and writes
// its results with four threads a token, through a scratch in shared memory, since with a
// thread a token every such access touched 32 lines.  (An option of the engine, not its default:
// the product's tiles are one round for the SMs at 2,048 tokens, so this epilogue hides behind
// nothing, and the library's product with the rotation kernel behind it measures faster there.)
//
// One CTA an SM walks over tiles (tile = blockIdx.x + i * gridDim.x; the tiles of one block of
// weight rows are neighbours, so that block is read from HBM once and from L2 after that).  Roles:
//   warp 0      TMA producer: x tile (16 KB) and W tile (32 KB) per 64-wide K block into a ring of
//               four stages (full / empty mbarriers)
//   warp 1      allocates all 512 TMEM columns (two accumulators of 256), issues tcgen05.mma
//               (128 x 256 x 16, four per stage), commits stages and accumulators
//   warps 2-9   epilogue: two warps per quarter of the TMEM lanes, each half of the columns, 16
//               at a time: tcgen05.ld, bias, SiLU*mul or rotation in fp32, bf16 / fp32 stores.
//               The epilogue of a tile runs while the next tile's products go into the other
//               accumulator.
// The gated product runs on CTA pairs (template parameter PAIR; see PB_BYTES_PAIR below): a
// cluster of two CTAs on a tile of 256 tokens, every role as above in both CTAs except that only
// the first CTA's warp 1 issues products (tcgen05.mma.cta_group::2, 256 x 256 x 16) and that its
// barriers count both CTAs' loads and both CTAs' epilogue threads.
// Every wait is bounded; a wait that runs out sets *err (1 producer, 2 MMA issuer, 3 epilogue)
// and the roles leave their loops, after which the CTA frees its tensor memory and returns.
#include "tc_common.cuh"

namespace gf {

#ifndef GF_PN
#define GF_PN 256
#endif
constexpr int PM = 128;                       // tokens per tile
constexpr int PN = GF_PN;                     // weight rows per tile (a multiple of 32, <= 256)
// as many stages as shared memory holds: 4 at 256 rows (5 at 224 rows measured no faster)
constexpr int PSTAGES = (225 * 1024) / (PM * BK * 2 + PN * BK * 2);
constexpr uint32_t PA_BYTES = PM * BK * 2;    // x tile of a stage
constexpr uint32_t PB_BYTES = PN * BK * 2;    // W tile of a stage
static_assert(PN % 32 == 0 && PN <= 256 && PSTAGES >= 2, "tile width");
constexpr int EPI_WARPS = 8;
constexpr int P_THREADS = (2 + EPI_WARPS) * 32;
constexpr uint32_t P_TMEM_COLS = 512;
// The same on CTA pairs (a cluster of two; tcgen05 .cta_group::2): a tile of 256 tokens x PN weight
// rows.  Each CTA brings its 128 tokens and HALF of the weight rows of a K block; one thread of
// the pair's first CTA issues products of 256 x PN x 16 that read both CTAs' shared memory and
// write 128 token rows into each CTA's tensor memory.  A CTA's tensor core then reads 8 KB of
// operands a product from shared memory instead of 12 KB (which is what bounds the single-CTA
// kernel), and a weight tile crosses from L2 to an SM once for 256 tokens instead of 128.
constexpr uint32_t PB_BYTES_PAIR = (PN / 2) * BK * 2;       // this CTA's half of the W tile
constexpr int PSTAGES_PAIR = (220 * 1024) / (PM * BK * 2 + (PN / 2) * BK * 2);

__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
// (addresses in the cluster's shared window: the barrier may be another CTA's)
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
// A TMA load into this CTA's shared memory whose bytes are counted by a barrier of the pair's
// first CTA (no multicast: each CTA fetches what it holds).
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t bar,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.cta_group::2 "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this offset in both CTAs of the pair once the products issued so far
// are complete
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;"
      ::"r"(smem_u32(bar)), "h"(both)
      : "memory");
}
// D fp32, A and B bf16, both K-major, M = 256 over the pair, N = bn
__host__ __device__ constexpr uint32_t umma_idesc_pair(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(256 >> 4) << 24);
}

constexpr int PEPI_STORE = 0;                 // out[m, n] = acc (+ bias[n])
constexpr int PEPI_GATED = 2;                 // out[m, n / 2] = silu(acc[m, n]) * acc[m, n + 1], n even
constexpr int PEPI_QKV = 3;                   // + bias, q and k heads rotated, k and v to the cache
// A warp's scratch: 32 rows of 64 bytes; the 16-byte pieces of a row are swapped by bits 1 and 2 of
// the row, so that neither a thread a row nor four threads a row meet a bank twice in one access.
constexpr int QKV_SCRATCH_WARP = 32 * 64;
__device__ __forceinline__ int scr_at(int row, int piece) {
  return row * 64 + ((piece ^ ((row >> 1) & 3)) << 4);
}

// What the q/k/v epilogue needs beside the product: rows [q heads | k heads | v heads] of `hd`
// channels; q and k are rotated by the angles of the token's position (table row: cos | sin over
// hd channels, half-rotation pairing j <-> j + hd / 2) after they have been rounded to bf16, as a
// rotation kernel behind the product would find them; k (rotated) and v also go to the token's
// slot of the paged cache ([slots][nkv][hd]; a negative slot is skipped).
struct QkvArgs {
  const float* rope;
  const int* positions;
  const int* slot_mapping;
  bf16* kpages;
  bf16* vpages;
  int nh, nkv, hd;
};

__device__ __forceinline__ float round_bf16(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}
__device__ __forceinline__ void store16_bf16(bf16* dst, const float (&v)[16]) {
#pragma unroll
  for (int j = 0; j < 16; j += 8) {
    __nv_bfloat162 p[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) p[u] = __floats2bfloat162_rn(v[j + 2 * u], v[j + 2 * u + 1]);
    *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(p);
  }
}

// eight of sixteen values, from `first`, as 16 bytes of bf16
__device__ __forceinline__ void store8_bf16(void* dst, const float (&v)[16], int first) {
  __nv_bfloat162 p[4];
#pragma unroll
  for (int u = 0; u < 4; ++u) p[u] = __floats2bfloat162_rn(v[first + 2 * u], v[first + 2 * u + 1]);
  *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(p);
}

template <int EPI, typename OUT, bool PAIR = false>
__global__ void __launch_bounds__(P_THREADS)
gemm_prefill_kernel(const __grid_constant__ CUtensorMap tmap_x,
                    const __grid_constant__ CUtensorMap tmap_w, const float* __restrict__ bias,
                    OUT* __restrict__ out, int ldo, int M, int N, int K, const QkvArgs qkv,
                    int* __restrict__ err) {
  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* tiles = (unsigned char*)(((uintptr_t)smem + 1023) & ~(uintptr_t)1023);
  constexpr int NST = PAIR ? PSTAGES_PAIR : PSTAGES;
  constexpr uint32_t B_BYTES = PAIR ? PB_BYTES_PAIR : PB_BYTES;
  constexpr uint32_t STAGE = PA_BYTES + B_BYTES;
  uint64_t* full = (uint64_t*)(tiles + NST * STAGE);
  uint64_t* empty = full + NST;
  uint64_t* acc_full = empty + NST;           // [2]
  uint64_t* acc_empty = acc_full + 2;         // [2]
  uint64_t* bias_ready = acc_empty + 2;       // the epilogue threads have staged a tile's bias
  uint32_t* tmem_slot = (uint32_t*)(bias_ready + 1);
  // the bias of a tile's PN columns, for the tile in either accumulator: with nearly all of the
  // SM's memory carved out as shared memory, a bias read from global memory in the epilogue's
  // inner loop goes to L2 every time
  float* bias_s = (float*)(tmem_slot + 4);    // [2][PN]
  // the q/k/v epilogue's scratch: 32 rows of 64 bytes (80 apart) for each epilogue warp, through
  // which it turns "a thread a token" into "four threads a token" and back (see there)
  unsigned char* scratch_s =
      (unsigned char*)(((uintptr_t)(bias_s + 2 * PN) + 15) & ~(uintptr_t)15);   // 16-byte pieces

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // a pair: the cluster walks over tiles of 2 * PM tokens, this CTA has rows rank * PM .. of them
  const uint32_t rank = PAIR ? cluster_rank() : 0u;
  const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  constexpr int TM = PAIR ? 2 * PM : PM;
  const int m_tiles = (M + TM - 1) / TM, n_tiles = (N + PN - 1) / PN;
  const int ntiles = m_tiles * n_tiles;
  const int nkb = (K + BK - 1) / BK;

  pdl_trigger();
  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) {
      mbar_init(full + s, PAIR ? 2 : 1);      // a pair: the first CTA's counts both CTAs' loads
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, (PAIR ? 2 : 1) * EPI_WARPS * 32);   // both CTAs' epilogue threads
    }
    mbar_init(bias_ready, EPI_WARPS * 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_x) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
  }
  if (warp == 1) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(tmem_slot)), "r"(P_TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                   ::"r"(smem_u32(tmem_slot)), "r"(P_TMEM_COLS)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync();                    // the peer's barriers exist before anything signals them
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      pdl_wait();                                      // x comes from the kernel in front
      int it = 0;                                      // K blocks issued so far, over all tiles
      bool ok = true;
      for (int tile = walker; tile < ntiles && ok; tile += walkers) {
        const int n0 = (tile / m_tiles) * PN + (PAIR ? (int)rank * (PN / 2) : 0);
        const int m0 = (tile % m_tiles) * TM + (int)rank * PM;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % NST;
          if (!mbar_wait(empty + s, ((it / NST) & 1) ^ 1, err, 1)) { ok = false; break; }
          unsigned char* a = tiles + s * STAGE;
          if (PAIR) {
            const uint32_t bar = peer_addr(smem_u32(full + s), 0);     // the first CTA's
            mbar_expect_tx_cluster(bar, STAGE);
            tma_load_2d_pair(a, &tmap_x, bar, kb * BK, m0);
            tma_load_2d_pair(a + PA_BYTES, &tmap_w, bar, kb * BK, n0);
          } else {
            mbar_expect_tx(full + s, STAGE);
            tma_load_2d(a, &tmap_x, full + s, kb * BK, m0);
            tma_load_2d(a + PA_BYTES, &tmap_w, full + s, kb * BK, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {                            // a pair: its first CTA issues for both
      // The whole warp walks through the K blocks; lane 0 issues the products.  The waits for
      // the stages are made AHEAD stages at a time, each by a lane of its own (see
      // mbar_wait_lanes): one after the other they took as long as the products themselves.
      constexpr uint32_t idesc = PAIR ? umma_idesc_pair(PN) : umma_idesc(PN);
      constexpr int AHEAD = PAIR ? NST / 2 : 1;      // (single CTAs: four stages, no gain measured)
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = walker; tile < ntiles && ok; tile += walkers, ++t) {
        const int buf = t & 1, use = t >> 1;
        // the epilogue must have read this accumulator's last tile (passes at once the first time)
        if (!mbar_wait(acc_empty + buf, (uint32_t)(use & 1) ^ 1u, err, 2)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t acc = tmem + (uint32_t)(buf * 256);
        for (int kb0 = 0; kb0 < nkb && ok; kb0 += AHEAD) {
          const int n = min(AHEAD, nkb - kb0);
          {
            const int mine = it + min(lane, n - 1);
            ok = mbar_wait_lanes(full + mine % NST, (uint32_t)(mine / NST) & 1u, lane < n, err, 2);
          }
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (lane == 0) {
            for (int j = 0; j < n; ++j) {
              const int s = (it + j) % NST;
              const uint32_t a = smem_u32(tiles + s * STAGE);
              const uint64_t ad = umma_desc(a), bd = umma_desc(a + PA_BYTES);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                const uint32_t accumulate = (kb0 + j > 0 || k > 0) ? 1u : 0u;
                if (PAIR)
                  umma_pair(acc, ad + (uint64_t)(k * UMMA_K * 2 >> 4),
                            bd + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, accumulate);
                else
                  umma(acc, ad + (uint64_t)(k * UMMA_K * 2 >> 4),
                       bd + (uint64_t)(k * UMMA_K * 2 >> 4), idesc, accumulate);
              }
              // the stage is free (in both CTAs of a pair) once these have read it
              if (PAIR) umma_commit_pair(empty + s);
              else umma_commit(empty + s);
            }
          }
          it += n;
        }
        if (ok && lane == 0) {                         // the tile's accumulator is complete
          if (PAIR) umma_commit_pair(acc_full + buf);
          else umma_commit(acc_full + buf);
        }
      }
    }
  } else {
    // epilogue: TMEM lanes (warp % 4) * 32 .. + 31 = tokens, columns half * 128 .. + 127
    const int e = warp - 2, q = warp & 3, half = e >> 2;
    pdl_wait();                                        // nothing is written before the kernel ahead is done
    // this thread has read its part of an accumulator (a pair: the first CTA's thread that
    // issues the products counts both CTAs' epilogue threads)
    auto acc_read = [&](int buf) {
      if (PAIR) mbar_arrive_cluster(peer_addr(smem_u32(acc_empty + buf), 0));
      else mbar_arrive(acc_empty + buf);
    };
    int t = 0;
    for (int tile = walker; tile < ntiles; tile += walkers, ++t) {
      const int buf = t & 1, use = t >> 1;
      const int n0 = (tile / m_tiles) * PN + half * (PN / 2);
      const int m = (tile % m_tiles) * TM + (int)rank * PM + q * 32 + lane;
      const float* bias_t = bias_s + buf * PN + half * (PN / 2);     // of this thread's columns
      if (EPI != PEPI_GATED && bias) {
        const int tn0 = (tile / m_tiles) * PN;
        for (int i = e * 32 + lane; i < PN; i += EPI_WARPS * 32)
          bias_s[buf * PN + i] = tn0 + i < N ? bias[tn0 + i] : 0.f;
        // every epilogue thread has written its part (a bounded wait like the others: a warp
        // that gave up does not leave the rest at a barrier); the warps are then at most a tile
        // apart, and the tiles alternate buffers
        mbar_arrive(bias_ready);
        if (!mbar_wait(bias_ready, (uint32_t)t & 1u, err, 3)) break;
      }
      // q/k/v: what the epilogue reads beside the accumulator is asked for before the wait for it
      const int rr = lane >> 2, pc = lane & 3;         // four threads a token: token rr (+ 8 i), piece pc
      int pos_t[4] = {0, 0, 0, 0}, slot_t[4] = {-1, -1, -1, -1}, slot_v[2] = {-1, -1};
      float4 tc[4], ts[4];                             // cos and sin of the chunk of channels to come
      auto load_table = [&](int j) {                   // channels j + 4 pc .. + 3 of tokens rr + 8 i
        const int hd = qkv.hd;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float* trow = qkv.rope + (size_t)pos_t[i] * hd + j + 4 * pc;
          tc[i] = __ldg(reinterpret_cast<const float4*>(trow));
          ts[i] = __ldg(reinterpret_cast<const float4*>(trow + (hd >> 1)));
        }
      };
      if (EPI == PEPI_QKV) {
        const int mm = m < M ? m : M - 1;
        const int pos_mine = qkv.positions[mm];
        const int slot_mine = m < M ? qkv.slot_mapping[mm] : -1;     // negative: nothing is cached
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          pos_t[i] = __shfl_sync(0xffffffffu, pos_mine, 8 * i + rr);
          slot_t[i] = __shfl_sync(0xffffffffu, slot_mine, 8 * i + rr);
        }
#pragma unroll
        for (int i = 0; i < 2; ++i) slot_v[i] = __shfl_sync(0xffffffffu, slot_mine, 16 * i + (lane >> 1));
        if (n0 / qkv.hd < qkv.nh + qkv.nkv) load_table(0);           // the first head is rotated
      }
      if (!mbar_wait(acc_full + buf, (uint32_t)(use & 1), err, 3)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * 256 + half * (PN / 2));
      if (EPI == PEPI_QKV) {
        // Whole heads of this thread's token: hd divides the half tile's 128 columns.  The
        // accumulator gives a thread one token's row, but a warp that reads the table or writes
        // `out` and the cache that way touches 32 lines with every instruction, and these, not
        // the bytes, are what the epilogue then waits for.  So the table is read, and the
        // results are written, with four threads a token (8 tokens x 64 bytes an instruction),
        // and the warp's scratch in shared memory turns one lay-out into the other.
        const int hd = qkv.hd, hh = hd >> 1;
        unsigned char* scr = scratch_s + (size_t)e * QKV_SCRATCH_WARP;
        const int m_w0 = m - lane;                     // the warp's first token
        bf16* outb = reinterpret_cast<bf16*>(out);
#pragma unroll 1
        for (int hb = 0; hb < PN / 2 && n0 + hb < N; hb += hd) {
          const int head = (n0 + hb) / hd;
          if (head >= qkv.nh + qkv.nkv) {             // a v head: bias, to `out` and to the cache
            const int vh = head - qkv.nh - qkv.nkv;
#pragma unroll 1
            for (int j = 0; j < hd; j += 16) {
              float v[16];
              __syncwarp();
              tmem_ld16(taddr + hb + j, v);
              if (bias) {
#pragma unroll
                for (int u = 0; u < 16; ++u) v[u] += bias_t[hb + j + u];
              }
              // (a row's two pieces go to its first or second half by bit 1 of the row: with two
              // threads a row, four rows are read at once)
              store8_bf16(scr + scr_at(lane, (lane & 2) + 0), v, 0);
              store8_bf16(scr + scr_at(lane, (lane & 2) + 1), v, 8);
              __syncwarp();
              // two threads a token: 16 tokens x 32 bytes an instruction
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int row = 16 * i + (lane >> 1), mr = m_w0 + row, col = j + 8 * (lane & 1);
                const uint4 piece =
                    *reinterpret_cast<const uint4*>(scr + scr_at(row, (row & 2) + (lane & 1)));
                if (mr < M) {
                  *reinterpret_cast<uint4*>(outb + (size_t)mr * ldo + n0 + hb + col) = piece;
                  if (slot_v[i] >= 0)
                    *reinterpret_cast<uint4*>(qkv.vpages +
                                              ((size_t)slot_v[i] * qkv.nkv + vh) * hd + col) = piece;
                }
              }
            }
          } else {                                    // a q or k head: bias, round, rotate
            const bool k_head = head >= qkv.nh;
#pragma unroll 1
            for (int j = 0; j < hh; j += 16) {
              // (cos and sin of this chunk were asked for a chunk ago, or before the accumulator
              // was waited for)
              float a[16], b[16];
              __syncwarp();
              tmem_ld16_async(taddr + hb + j, a);
              tmem_ld16_async(taddr + hb + hh + j, b);
              tmem_ld_wait();
              float cc[16], ss[16];
#pragma unroll
              for (int i = 0; i < 4; ++i)
                *reinterpret_cast<float4*>(scr + scr_at(8 * i + rr, pc)) = tc[i];
              __syncwarp();
#pragma unroll
              for (int u = 0; u < 4; ++u)
                *reinterpret_cast<float4*>(cc + 4 * u) =
                    *reinterpret_cast<const float4*>(scr + scr_at(lane, u));
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i)
                *reinterpret_cast<float4*>(scr + scr_at(8 * i + rr, pc)) = ts[i];
              __syncwarp();
#pragma unroll
              for (int u = 0; u < 4; ++u)
                *reinterpret_cast<float4*>(ss + 4 * u) =
                    *reinterpret_cast<const float4*>(scr + scr_at(lane, u));
              __syncwarp();
              // the next chunk's, or (the table is the same for every head) the next head's first
              load_table(j + 16 < hh ? j + 16 : 0);
#pragma unroll
              for (int u = 0; u < 16; ++u) {
                const float x = round_bf16(a[u] + (bias ? bias_t[hb + j + u] : 0.f));
                const float y = round_bf16(b[u] + (bias ? bias_t[hb + hh + j + u] : 0.f));
                a[u] = x * cc[u] - y * ss[u];
                b[u] = x * ss[u] + y * cc[u];
              }
              // this token's 16 + 16 results as 64 bytes of its scratch row, then four threads a
              // token: pieces 0, 1 are channels j .. j + 15, pieces 2, 3 channels hh + j .. + 15
              store8_bf16(scr + scr_at(lane, 0), a, 0);
              store8_bf16(scr + scr_at(lane, 1), a, 8);
              store8_bf16(scr + scr_at(lane, 2), b, 0);
              store8_bf16(scr + scr_at(lane, 3), b, 8);
              __syncwarp();
              const int col = pc < 2 ? j + 8 * pc : hh + j + 8 * (pc - 2);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int row = 8 * i + rr, mr = m_w0 + row;
                const uint4 piece = *reinterpret_cast<const uint4*>(scr + scr_at(row, pc));
                if (mr < M) {
                  *reinterpret_cast<uint4*>(outb + (size_t)mr * ldo + n0 + hb + col) = piece;
                  if (k_head && slot_t[i] >= 0)
                    *reinterpret_cast<uint4*>(qkv.kpages + ((size_t)slot_t[i] * qkv.nkv +
                                                            (head - qkv.nh)) * hd + col) = piece;
                }
              }
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        acc_read(buf);
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < PN / 2; c += 16) {
        float v[16];
        __syncwarp();                                  // the load below wants the whole warp
        if (nkb > 0) {
          tmem_ld16(taddr + c, v);
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0.f;
        }
        if (c == PN / 2 - 16) {                        // the last read of this accumulator
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          acc_read(buf);
        }
        const int n = n0 + c;
        if (m >= M || n >= N) continue;
        if (EPI == PEPI_STORE) {
          if (bias) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += bias_t[c + j];
          }
          OUT* dst = out + (size_t)m * ldo + n;
          if (sizeof(OUT) == 2) {
#pragma unroll
            for (int j = 0; j < 16; j += 8) {
              if (n + j >= N) break;                   // N is a multiple of 8
              __nv_bfloat162 p[4];
#pragma unroll
              for (int u = 0; u < 4; ++u) p[u] = __floats2bfloat162_rn(v[j + 2 * u], v[j + 2 * u + 1]);
              *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(p);
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; j += 4) {
              if (n + j >= N) break;
              *reinterpret_cast<float4*>(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
          }
        } else {
          // (gate, up) in neighbouring columns, both rounded to bf16 first as a product's output
          // would be; 8 results (N is a multiple of 16 here)
          __nv_bfloat162 p[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float z[2];
#pragma unroll
            for (int w = 0; w < 2; ++w) {
              const float g = __bfloat162float(__float2bfloat16_rn(v[4 * u + 2 * w]));
              const float up = __bfloat162float(__float2bfloat16_rn(v[4 * u + 2 * w + 1]));
              z[w] = g * (1.0f / (1.0f + expf(-g))) * up;
            }
            p[u] = __floats2bfloat162_rn(z[0], z[1]);
          }
          *reinterpret_cast<uint4*>(out + (size_t)m * ldo + (n >> 1)) =
              *reinterpret_cast<const uint4*>(p);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (PAIR) cluster_sync();                    // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                   "r"(P_TMEM_COLS)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                   "r"(P_TMEM_COLS)
                   : "memory");
  }
}

template <int EPI, typename OUT, bool PAIR = false>
static int launch_prefill(const CUtensorMap& mx, const CUtensorMap& mw, const float* bias, void* out,
                          int ldo, int M, int N, int K, int* err, int ctas, cudaStream_t st,
                          const QkvArgs& qkv = QkvArgs{}) {
  constexpr int NST = PAIR ? PSTAGES_PAIR : PSTAGES;
  const size_t smem = 1024 + (size_t)NST * (PA_BYTES + (PAIR ? PB_BYTES_PAIR : PB_BYTES)) +
                      (2 * NST + 5) * sizeof(uint64_t) + 32 + 2 * PN * sizeof(float) +
                      (EPI == PEPI_QKV ? EPI_WARPS * QKV_SCRATCH_WARP : 0);
  auto k = gemm_prefill_kernel<EPI, OUT, PAIR>;
  static OncePerDevice attrs;                        // (of this instantiation of the launcher)
  if (int rc = attrs.run([&] {
        return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      }))
    return rc;
  if (PAIR)
    return launch_kernel_cluster_dims(k, dim3(ctas & ~1), dim3(P_THREADS), smem, st, 2, true, mx, mw,
                                      bias, (OUT*)out, ldo, M, N, K, qkv, err);
  return launch_kernel(k, dim3(ctas), dim3(P_THREADS), smem, st, mx, mw, bias, (OUT*)out, ldo, M,
                       N, K, qkv, err);
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

// x [M, K] bf16 (row stride ldx), w [N, K] bf16 contiguous, bias fp32 [N] or null.
// epi 0: out [M, N] (row stride ldo) bf16 or fp32 = x w^T (+ bias); epi 2: w rows interleaved
// (gate_i, up_i), out [M, N / 2] bf16 = silu(gate) * up.  `ctas`: CTAs to launch (0: one an SM).
// -6: a shape or alignment this kernel does not take (the caller uses another product).
// `pair`: on CTA pairs (tiles of 256 tokens; see the top of the file).
GF_EXPORT int gf_gemm_prefill(const void* x, int ldx, const void* w, const void* bias, void* out,
                              int ldo, int M, int N, int K, int epi, int out_f32, int ctas,
                              int* err, void* stream, int pair) {
  if (M <= 0 || N <= 0) return 0;
  if (K < 8 || K % 8 || ldx % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) ||
      ((uintptr_t)out & 15))
    return -6;
  if (epi == PEPI_GATED ? (N % 16 || ldo % 8 || out_f32) : (epi != PEPI_STORE || N % 8 ||
                                                            ldo % (out_f32 ? 4 : 8)))
    return -6;
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, ldx, PM)) return -6;
  if (!make_map(&mw, w, N, K, K, pair ? PN / 2 : PN)) return -6;
  const int tm = pair ? 2 * PM : PM;
  const int ntiles = ((M + tm - 1) / tm) * ((N + PN - 1) / PN);
  int sms = 148;
  {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) == cudaSuccess &&
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
      sms = v;
  }
  if (ctas <= 0 || ctas > sms) ctas = sms;
  if (pair) {
    if (ctas > 2 * ntiles) ctas = 2 * ntiles;
    ctas &= ~1;
    if (ctas < 2) return -6;
  } else if (ctas > ntiles) {
    ctas = ntiles;
  }
  auto st = (cudaStream_t)stream;
  if (pair) {
    if (epi == PEPI_GATED)
      return launch_prefill<PEPI_GATED, bf16, true>(mx, mw, nullptr, out, ldo, M, N, K, err, ctas,
                                                    st);
    if (out_f32)
      return launch_prefill<PEPI_STORE, float, true>(mx, mw, (const float*)bias, out, ldo, M, N, K,
                                                     err, ctas, st);
    return launch_prefill<PEPI_STORE, bf16, true>(mx, mw, (const float*)bias, out, ldo, M, N, K,
                                                  err, ctas, st);
  }
  if (epi == PEPI_GATED)
    return launch_prefill<PEPI_GATED, bf16>(mx, mw, nullptr, out, ldo, M, N, K, err, ctas, st);
  if (out_f32)
    return launch_prefill<PEPI_STORE, float>(mx, mw, (const float*)bias, out, ldo, M, N, K, err,
                                             ctas, st);
  return launch_prefill<PEPI_STORE, bf16>(mx, mw, (const float*)bias, out, ldo, M, N, K, err, ctas,
                                          st);
}

// The q/k/v product of prompt portions with what follows it in its epilogue: x [M, K] bf16, w
// [(nh + 2 nkv) * hd, K] bf16 (q heads, k heads, v heads), bias fp32 or null; out [M, N] bf16
// receives q and k rotated and v; k (rotated) and v also go to slot slot_mapping[m] of the paged
// cache.  rope: [positions][hd] fp32, cos | sin (the whole head is rotated).  Head sizes 64 and
// 128.  -6: not served.
GF_EXPORT int gf_gemm_prefill_qkv(const void* x, int ldx, const void* w, const void* bias,
                                  void* out, int ldo, int M, int K, int nh, int nkv, int hd,
                                  const float* rope, const int* positions,
                                  const int* slot_mapping, void* kpages, void* vpages, int ctas,
                                  int* err, void* stream) {
  const int N = (nh + 2 * nkv) * hd;
  if (M <= 0 || N <= 0) return 0;
  if ((hd != 64 && hd != 128) || !rope || !positions || !slot_mapping || !kpages || !vpages)
    return -6;
  if (K < 8 || K % 8 || ldx % 8 || ldo % 8 || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) ||
      ((uintptr_t)out & 15) || ((uintptr_t)kpages & 15) || ((uintptr_t)vpages & 15))
    return -6;
  CUtensorMap mx, mw;
  if (!make_map(&mx, x, M, K, ldx, PM)) return -6;
  if (!make_map(&mw, w, N, K, K, PN)) return -6;
  const int ntiles = ((M + PM - 1) / PM) * ((N + PN - 1) / PN);
  int sms = 148, dev = 0, v = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
    sms = v;
  if (ctas <= 0 || ctas > sms) ctas = sms;
  if (ctas > ntiles) ctas = ntiles;
  const QkvArgs args{rope, positions, slot_mapping, (bf16*)kpages, (bf16*)vpages, nh, nkv, hd};
  return launch_prefill<PEPI_QKV, bf16>(mx, mw, (const float*)bias, out, ldo, M, N, K, err, ctas,
                                        (cudaStream_t)stream, args);
}
