// Prefill attention on the 5th-generation tensor cores: varlen, causal (+ sliding window), GQA,
// over the paged cache.  Compiled for one head size (-DGF_HEAD_DIM = 64 or 128).
//
// One CTA owns 128 query rows of one head of one request.  Keys are visited in tiles of 128.  For a
// tile j:   S = Q K_j^T      tcgen05.mma, A = Q and B = K_j in shared memory (K-major, 128B
//                             swizzle, written by TMA), D = S in tensor memory (128 lanes x 128 fp32)
//           P = softmax part  four warps, one thread per query row: tcgen05.ld of its row of S
//                             (S is double buffered: S_{j+1} is computed meanwhile), running
//                             maximum and sum in fp32, P rounded to bf16 into shared memory
//           O += P V_j        tcgen05.mma, A = P (K-major), B = V_j as stored ([key][channel], that
//                             is MN-major), D = O in tensor memory (128 lanes x HD fp32)
// The accumulator O is rescaled in tensor memory only when a row's maximum has grown by more than
// 2^8 since the last rescale (the probabilities then stay below 2^8, well inside bf16 and fp32).
// K and V tiles come page by page through TMA: the cache of one layer is a 2-D tensor
// [token slots, kv_heads * HD]; a page is a box of page_size rows; pages past the request's end are
// loaded from out-of-range coordinates, which TMA fills with zeros.
//
// Warps: 0..3 = TMA loaders (K: 0-1, V: 2-3; every lane issues one box), 4 = tensor-memory
// allocation and MMA issue (one thread), 5..12 = softmax and epilogue (two threads per query row).  The reference's prefill kernel is a 64x64 mma.sync
// flash loop with S, P and the row maximum held in bf16
// (ginfer/core/op/kernels/cuda/page_attn_kernel/flash_gqa_varlen_kernel.cu:420-512).
//
// Every wait on an mbarrier is bounded; when one runs out, the waiter records a code in *err, an
// abort flag in shared memory tells the other roles to leave their loops, all meet at the final
// barrier and tensor memory is freed.
#include <cuda.h>

#include "common.cuh"

#ifndef GF_HEAD_DIM
#define GF_HEAD_DIM 128
#endif

namespace gf {

constexpr int HD = GF_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
constexpr int QT = 128;                    // query rows per CTA = TMEM lanes
constexpr int KT = 128;                    // keys per tile
constexpr int HALVES = HD / 64;            // 64-channel swizzle atoms per row
constexpr int K_STAGES = HD == 128 ? 3 : 4;   // K_j is free as soon as S_j is computed
constexpr int V_STAGES = HD == 128 ? 2 : 3;   // V_j is free once O += P_j V_j is complete
constexpr int NTHREADS = 416;              // four loader warps, MMA warp, eight softmax warps
constexpr uint32_t ATOM_BYTES = 128 * 64 * 2;            // a [128][64] bf16 tile: 16 KB
constexpr uint32_t Q_BYTES = HALVES * ATOM_BYTES;
constexpr uint32_t K_BYTES = HALVES * ATOM_BYTES;        // [128 keys][HD]
constexpr uint32_t V_BYTES = HALVES * ATOM_BYTES;
constexpr uint32_t P_BYTES = 2 * ATOM_BYTES;             // [128 rows][128 keys]
constexpr uint32_t TMEM_COLS = 512;                      // S0: 0..127, S1: 128..255, O: 256..
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float kRescaleStep = 8.f;        // log2 units a maximum may grow before O is rescaled

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; gives up early when another role has raised the abort flag.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* err, int code) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if (spin > 64) {
      if (*abort_flag) return false;
      __nanosleep(32);
    }
  }
  *abort_flag = 1;
  if (err) atomicExch(err, code);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// Shared-memory operand descriptors (sm_100 version, 128-byte swizzle).
// K-major [rows][64]: rows 128 B apart, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major (V as stored: [key][channel]): a 128-byte row holds 64 channels of one key; 8 keys make
// a 1024-byte group (stride byte offset); the next 64 channels start one atom (16 KB) further on
// (leading byte offset).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(ATOM_BYTES >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D fp32, A and B bf16, M = 128, N = n; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t id,
                                     uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(id), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
               ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// The registers written by tmem_ld32 hold data only after this.
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])),
      "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])),
      "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
      "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])),
      "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])),
      "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
      "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
      "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])),
      "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])),
      "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x on the FMA and integer pipes, for a share of a tile's exponentials: the special-function
// unit gives 16 results a cycle and SM, and a tile of 128 x 128 scores wants 16,384 of them.
// x = n + f with n the nearest integer (read from the low mantissa bits of x + 1.5 * 2^23) and
// f in [-0.5, 0.5]; 2^f by a cubic whose largest relative error there is 7.5e-5 (the result is
// rounded to bf16, 3.9e-3, right after); n is added to the exponent field.  x is clamped at -125,
// so that the result stays a normal number (about 2e-38: nothing, beside a row's largest term).
// Off unless the build asks for it: shares of 1/8, 1/4, 1/3 and 1/2 measured 6.51, 6.60, 6.68 and
// 6.55 ms a 2,048-token prefill of the 1.5B shape against 6.54 ms without, all within the noise.
#ifndef GF_POLY_EXP_EVERY
#define GF_POLY_EXP_EVERY 0          // every n-th exponential of an unmasked tile; 0: none
#endif
__device__ __forceinline__ float poly_exp2(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;
  const float f = x - (t - 12582912.f);
  float p = fmaf(0.05517132207751274f, f, 0.24261054396629333f);
  p = fmaf(p, f, 0.6932609677314758f);
  p = fmaf(p, f, 0.9999281167984009f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct Barriers {
  uint64_t q_full;
  uint64_t q_empty;       // the item's last S product has read Q
  uint64_t k_full[K_STAGES];
  uint64_t k_empty[K_STAGES];
  uint64_t v_full[V_STAGES];
  uint64_t v_empty[V_STAGES];
  uint64_t s_full[2];     // S_j is complete in tensor memory (buffer j % 2)
  uint64_t p_ready;       // P_j is in shared memory and O is rescaled (256 arrivals)
  uint64_t max_ready;     // both halves of every row have posted their maximum (256 arrivals)
  uint64_t pv_done;       // O += P_j V_j is complete
  uint64_t o_free;        // the softmax warps have read an item's O out (256 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  float row_max[2][2][QT];   // [tile parity][half][row]
};

// One work item: 128 query rows of one head of one request, and the key tiles they see.
struct Item {
  int b, head, r0, rows, q_begin, pos0, key_lo, p_last, j0, ntiles, kvh;
};

__global__ void __launch_bounds__(NTHREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                       const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v,
                       const int* __restrict__ block_table, int table_stride,
                       const int* __restrict__ cu_seqlens_q, const int* __restrict__ kv_lens,
                       bf16* __restrict__ out, int nh, int nkv, int page_size, int window,
                       float scale_log2, int oob_row, int q_tiles, int B,
                       int* __restrict__ err, long long* __restrict__ dbg) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // the kernel has no static shared memory, so the dynamic part starts at the aligned base; the
  // swizzled tiles need that (checked below: a misaligned base ends the CTA with an error code)
  unsigned char* q_s = smem_raw;
  unsigned char* k_s = q_s + Q_BYTES;                      // [K_STAGES][K_BYTES]
  unsigned char* v_s = k_s + K_STAGES * K_BYTES;           // [V_STAGES][V_BYTES]
  unsigned char* p_s = v_s + V_STAGES * V_BYTES;
  Barriers* bars = reinterpret_cast<Barriers*>(p_s + P_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // optional time stamps of the first CTA's first item (dbg: 16 slots per tile per role)
  bool trace = dbg != nullptr && blockIdx.x == 0;
#define GF_STAMP(role, i, slot) \
  if (trace && (i) < 32) dbg[((role) * 32 + (i)) * 8 + (slot)] = clock64()  /* dbg: 3 * 32 * 8 */
  // with dbg: every CTA also leaves (start ns, end ns, SM) behind the first CTA's stamps
  const int cta_lin = blockIdx.x;
  if (dbg && threadIdx.x == 0) {
    unsigned long long t;
    unsigned int sm;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    dbg[768 + cta_lin * 4] = (long long)t;
    dbg[768 + cta_lin * 4 + 2] = sm;
  }
  pdl_trigger();
  pdl_wait();
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && err) atomicExch(err, 12);
    return;
  }
  // The CTAs (one an SM) walk over the work items.  Items are numbered heads fastest, then query
  // tiles from the last (heaviest: most keys under the causal mask) to the first, then requests;
  // CTA c takes items c, 2G - 1 - c, 2G + c, ... (G CTAs): the CTAs that got the lightest items of
  // one round get the heaviest of the next.  Barrier phases run on over the items (every role
  // counts tiles and items for itself), so the loads and the first S product of the next item
  // overlap the last P V, the read-out and the stores of this one.
  const int items = nh * q_tiles * B;
  auto item_of = [&](int n, Item& it) -> int {   // 0: no more items, 1: it, 2: an empty item
    const int G = gridDim.x;
    const int idx = n * G + ((n & 1) ? G - 1 - (int)blockIdx.x : (int)blockIdx.x);
    if (idx >= items) return 0;
    it.head = idx % nh;
    const int rest = idx / nh;
    it.b = rest / q_tiles;
    it.r0 = (q_tiles - 1 - rest % q_tiles) * QT;
    it.q_begin = cu_seqlens_q[it.b];
    const int q_len = cu_seqlens_q[it.b + 1] - it.q_begin;
    if (it.r0 >= q_len) return 2;
    const int kv_len = kv_lens[it.b];
    it.pos0 = kv_len - q_len;
    it.kvh = it.head / (nh / nkv);
    it.rows = min(QT, q_len - it.r0);
    const int p_first = it.pos0 + it.r0;
    it.p_last = it.pos0 + it.r0 + it.rows - 1;
    it.key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    it.j0 = it.key_lo / KT;
    it.ntiles = it.p_last / KT - it.j0 + 1;
    return 1;
  };

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    mbar_init(&bars->q_empty, 1);
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(&bars->k_full[s], 2);          // one arrival (with its byte count) per loader warp
      mbar_init(&bars->k_empty[s], 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(&bars->v_full[s], 2);
      mbar_init(&bars->v_empty[s], 1);
    }
    mbar_init(&bars->s_full[0], 1);
    mbar_init(&bars->s_full[1], 1);
    mbar_init(&bars->p_ready, 256);
    mbar_init(&bars->max_ready, 256);
    mbar_init(&bars->pv_done, 1);
    mbar_init(&bars->o_free, 256);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_v) : "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&bars->tmem_base)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = bars->tmem_base;
  const uint32_t tmem_s = tmem, tmem_o = tmem + 256;          // S buffer b at tmem_s + 128 * b

  if (warp < 4) {
    // ------------------------------------------------------------------ loaders
    // Four warps: warps 0-1 bring K tiles, warps 2-3 V tiles, each every other box of its
    // operand (a box = one page x 64 channels; issuing a TMA copy costs its thread ~80 cycles and
    // the lanes of a warp issue one after the other, so one warp alone could not keep up with
    // 16-token pages).  The block-table look-ups of tile i + 1 are made while tile i's boxes are
    // under way.
    const bool is_v = warp >= 2;
    const int part = warp & 1;
    const int pages_per_tile = KT / page_size;
    const int ops = pages_per_tile * HALVES;                   // boxes per tile of one operand
    const int my_ops = (ops - part + 1) / 2;                   // boxes part, part + 2, ...
    constexpr int MAX_OPS = ((KT / 8) * HALVES / 2 + 31) / 32; // page sizes down to 8
    const int nstages = is_v ? V_STAGES : K_STAGES;
    const uint32_t tile_bytes = is_v ? V_BYTES : K_BYTES;
    unsigned char* ring = is_v ? v_s : k_s;
    uint64_t* full = is_v ? bars->v_full : bars->k_full;
    uint64_t* empty = is_v ? bars->v_empty : bars->k_empty;
    const CUtensorMap* map = is_v ? &tmap_v : &tmap_k;
    const uint32_t my_bytes = (uint32_t)my_ops * (uint32_t)page_size * 128u;
    int cnt = 0, seq = 0;                                      // tiles and items so far
    bool go = true;
    Item it;
    for (int n = 0; go; ++n) {
      const int kind = item_of(n, it);
      if (kind == 0) break;
      if (kind == 2) continue;
      const int* tbl = block_table + (size_t)it.b * table_stride;
      if (warp == 0 && lane == 0) {
        // Q's buffer is free once the last S product of the item before has read it
        if (!mbar_wait(&bars->q_empty, (uint32_t)(seq & 1) ^ 1u, abort_flag, err, 13)) break;
        mbar_expect_tx(&bars->q_full, Q_BYTES);
        for (int h = 0; h < HALVES; ++h)
          tma_load_2d(q_s + h * ATOM_BYTES, &tmap_q, &bars->q_full, it.head * HD + h * 64,
                      it.q_begin + it.r0);
      }
      int rows_next[MAX_OPS];
      auto lookup = [&](int i) {
        const int key0 = (it.j0 + i) * KT;
#pragma unroll
        for (int u = 0; u < MAX_OPS; ++u) {
          const int op = part + 2 * (lane + 32 * u);
          rows_next[u] = oob_row;
          if (op < ops && i < it.ntiles) {
            const int c = key0 + (op / HALVES) * page_size;    // first key of this page
            // pages past the request's last key (or wholly before the window) come from an
            // out-of-range row: TMA fills them with zeros
            if (c <= it.p_last && c + page_size > it.key_lo) {
              const int page = tbl[c / page_size];
              if (page >= 0) rows_next[u] = page * page_size;
            }
          }
        }
      };
      lookup(0);
      for (int i = 0; i < it.ntiles; ++i, ++cnt) {
        int rows_now[MAX_OPS];
#pragma unroll
        for (int u = 0; u < MAX_OPS; ++u) rows_now[u] = rows_next[u];
        const int st = cnt % nstages;
        int ok = 1;
        if (lane == 0) {
          if (warp == 0) { GF_STAMP(2, i, 0); }
          ok = mbar_wait(&empty[st], ((cnt / nstages) & 1) ^ 1, abort_flag, err, 1);
          if (ok && my_bytes) mbar_expect_tx(&full[st], my_bytes);
          else if (ok) mbar_arrive(&full[st]);
          if (warp == 0) { GF_STAMP(2, i, 1); }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { go = false; break; }
#pragma unroll
        for (int u = 0; u < MAX_OPS; ++u) {
          const int op = part + 2 * (lane + 32 * u);
          if (op < ops) {
            const int pg = op / HALVES, h = op - pg * HALVES;
            tma_load_2d(ring + (size_t)st * tile_bytes + h * ATOM_BYTES +
                            (size_t)pg * page_size * 128,
                        map, &full[st], it.kvh * HD + h * 64, rows_now[u]);
          }
        }
        if (warp == 0 && lane == 0) { GF_STAMP(2, i, 2); }
        lookup(i + 1);                                          // overlaps the next wait
      }
      ++seq;
      trace = false;
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t id_qk = idesc(KT, false), id_pv = idesc(HD, true);
      const uint32_t qa = smem_u32(q_s), pa = smem_u32(p_s);
      int cnt = 0, seq = 0;                                    // tiles and items so far
      bool ok = true;
      Item it;
      for (int n = 0; ok; ++n) {
        const int kind = item_of(n, it);
        if (kind == 0) break;
        if (kind == 2) continue;
        const int c0 = cnt;                                    // the item's first tile
        ok = mbar_wait(&bars->q_full, (uint32_t)(seq & 1), abort_flag, err, 2);
        // S_i = Q K_i^T into S buffer (c0 + i) % 2: issued one tile ahead of P V, so that the
        // tensor core works on tile i + 1 while the softmax warps work on tile i
        auto issue_qk = [&](int i) -> bool {
          const int c = c0 + i, s = c % K_STAGES;
          if (!mbar_wait(&bars->k_full[s], (c / K_STAGES) & 1, abort_flag, err, 3)) return false;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t ka = smem_u32(k_s + s * K_BYTES);
#pragma unroll
          for (int k = 0; k < HD / 16; ++k) {
            const uint32_t off = (k / 4) * ATOM_BYTES + (k % 4) * 32;   // 16 channels = 32 bytes
            umma(tmem_s + 128 * (c & 1), desc_kmajor(qa + off), desc_kmajor(ka + off), id_qk,
                 k > 0 ? 1u : 0u);
          }
          umma_commit(&bars->k_empty[s]);       // K_i may be overwritten once S_i is computed
          umma_commit(&bars->s_full[c & 1]);
          if (i == it.ntiles - 1) umma_commit(&bars->q_empty);   // Q has been read for the last time
          return true;
        };
        if (ok) ok = issue_qk(0);
        for (int i = 0; i < it.ntiles && ok; ++i) {
          const int c = c0 + i, s = c % V_STAGES;
          // S buffer (c + 1) % 2 held the tile before this one: the softmax warps were done with
          // it before they announced its P, which this thread waited for in the last round
          GF_STAMP(1, i, 0);
          if (i + 1 < it.ntiles) ok = issue_qk(i + 1);
          if (!ok) break;
          GF_STAMP(1, i, 1);
          ok = mbar_wait(&bars->v_full[s], (c / V_STAGES) & 1, abort_flag, err, 9);
          GF_STAMP(1, i, 2);
          if (ok) ok = mbar_wait(&bars->p_ready, c & 1, abort_flag, err, 4);
          // the first P V of an item overwrites O: the item before must have been read out
          if (ok && i == 0)
            ok = mbar_wait(&bars->o_free, (uint32_t)(seq & 1) ^ 1u, abort_flag, err, 14);
          if (!ok) break;
          GF_STAMP(1, i, 3);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t va = smem_u32(v_s + s * V_BYTES);
#pragma unroll
          for (int k = 0; k < KT / 16; ++k) {
            const uint32_t poff = (k / 4) * ATOM_BYTES + (k % 4) * 32;  // 16 keys along P's rows
            const uint32_t voff = k * 16 * 128;                         // 16 keys = 16 rows of V
            umma(tmem_o, desc_kmajor(pa + poff), desc_mnmajor(va + voff), id_pv,
                 (i > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&bars->v_empty[s]);         // V_i may be overwritten
          umma_commit(&bars->pv_done);            // O holds tiles 0 .. i
          GF_STAMP(1, i, 4);
        }
        cnt = c0 + it.ntiles;
        ++seq;
        trace = false;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    // Eight warps: two threads per query row, each with 64 of the tile's 128 keys (and half of
    // O's channels), so that every scheduler has two warps to switch between.  The two threads of
    // a row agree on the row maximum through shared memory and an mbarrier (a bounded wait; a
    // named barrier could not be left if the other thread gave up).
    const int qd = warp & 3;                                   // TMEM lane quarter of this warp
    const int half = (warp - 5) >> 2;                          // which 64 keys / which channels
    const int r = qd * 32 + lane;                              // query row of this thread
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    int cnt = 0, mr = 0;                                       // tiles, and uses of max_ready
    bool ok = true;
    Item it;
    for (int n = 0; ok; ++n) {
      const int kind = item_of(n, it);
      if (kind == 0) break;
      if (kind == 2) continue;
      const int c0 = cnt;
      const int p = it.pos0 + it.r0 + r;                       // this row's position
      const bool live = r < it.rows;
      const int lo = window > 0 ? max(0, p - window + 1) : 0;
      float m_used = -INFINITY;        // the maximum the accumulated P and l are scaled by
      float l = 0.f;                   // this thread's half of the row sum
      for (int i = 0; i < it.ntiles; ++i) {
        const int c = c0 + i;
        const bool tr = r == 0 && half == 0;
        if (tr) { GF_STAMP(0, i, 0); }
        ok = mbar_wait(&bars->s_full[c & 1], (c >> 1) & 1, abort_flag, err, 5);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tr) { GF_STAMP(0, i, 1); }
        const int col0 = (it.j0 + i) * KT + 64 * half;         // first key of this thread's half
        // every row of this warp sees all of these keys: no comparisons
        const int wp0 = it.pos0 + it.r0 + qd * 32;
        const bool interior = col0 + 63 <= wp0 && qd * 32 + 32 <= it.rows &&
                              (window <= 0 || col0 >= wp0 + 31 - window + 1);
        float v[2][32];
        const uint32_t srow = tmem_s + 128 * (c & 1) + 64 * half + lane_addr;
        tmem_ld32(srow, v[0]);
        tmem_ld32(srow + 32, v[1]);
        tmem_ld_wait();
        if (tr) { GF_STAMP(0, i, 2); }
        // four running maxima (and four sums below) instead of one chain of dependent operations
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (interior) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int k = 0; k < 32; ++k) mx4[k & 3] = fmaxf(mx4[k & 3], v[cc][k]);
        } else {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int key = col0 + 32 * cc + k;
              v[cc][k] = (live && key >= lo && key <= p) ? v[cc][k] : -INFINITY;
              mx4[k & 3] = fmaxf(mx4[k & 3], v[cc][k]);
            }
        }
        float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // the row's maximum over both halves
        bars->row_max[mr & 1][half][r] = mx;
        mbar_arrive(&bars->max_ready);
        ok = mbar_wait(&bars->max_ready, mr & 1, abort_flag, err, 10);
        if (!ok) break;
        if (tr) { GF_STAMP(0, i, 3); }
        mx = fmaxf(mx, bars->row_max[mr & 1][half ^ 1][r]) * scale_log2;   // scale > 0
        ++mr;
        // lazy rescale: keep the old reference maximum unless the row's maximum outgrew it
        float m_new = m_used;
        if (mx > m_used + kRescaleStep || m_used == -INFINITY) m_new = fmaxf(m_used, mx);
        const float corr = (m_new == m_used) ? 1.f
                           : (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new));
        const float msub = m_new == -INFINITY ? 0.f : m_new;
        // probabilities (in place) and the row sum, while P V of the tile before may still run
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        if (GF_POLY_EXP_EVERY > 0 && interior) {
          // no key of this tile is masked for this warp: every score is finite
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const float x = fmaf(v[cc][k], scale_log2, -msub);
              const float e = (GF_POLY_EXP_EVERY > 0 &&
                               k % (GF_POLY_EXP_EVERY > 0 ? GF_POLY_EXP_EVERY : 1) ==
                                   GF_POLY_EXP_EVERY - 1)
                                  ? poly_exp2(x)
                                  : fast_exp2(x);
              v[cc][k] = e;
              sum4[k & 3] += e;
            }
        } else {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const float e = fast_exp2(fmaf(v[cc][k], scale_log2, -msub));
              v[cc][k] = e;
              sum4[k & 3] += e;
            }
        }
        const float sum = (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        if (tr) { GF_STAMP(0, i, 4); }
        // O and the P buffer are free once P V of the tile before is complete (the item's first
        // tile: the epilogue of the item before has waited for its last P V already)
        if (i > 0) {
          ok = mbar_wait(&bars->pv_done, (c - 1) & 1, abort_flag, err, 6);
          if (!ok) break;
          if (tr) { GF_STAMP(0, i, 5); }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (__any_sync(0xffffffffu, corr != 1.f)) {          // this thread's half of O's row
#pragma unroll 1
            for (int cc = 0; cc < HD / 2; cc += 32) {
              float o[32];
              tmem_ld32(tmem_o + lane_addr + half * (HD / 2) + cc, o);
              tmem_ld_wait();
#pragma unroll
              for (int k = 0; k < 32; ++k) o[k] *= corr;
              tmem_st32(tmem_o + lane_addr + half * (HD / 2) + cc, o);
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          }
        }
        l = l * corr + sum;
        m_used = m_new;
        // P (bf16, K-major with 128-byte swizzle) -> shared memory: keys 64 * half .. + 63 are
        // atom `half`, eight 16-byte chunks per row
        unsigned char* prow = p_s + half * ATOM_BYTES + (size_t)r * 128;
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int ch = 0; ch < 4; ++ch) {                     // 8 keys = one 16-byte chunk
            const int chunk = cc * 4 + ch;
            uint4 w;
            w.x = pack_bf16(v[cc][ch * 8 + 0], v[cc][ch * 8 + 1]);
            w.y = pack_bf16(v[cc][ch * 8 + 2], v[cc][ch * 8 + 3]);
            w.z = pack_bf16(v[cc][ch * 8 + 4], v[cc][ch * 8 + 5]);
            w.w = pack_bf16(v[cc][ch * 8 + 6], v[cc][ch * 8 + 7]);
            *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = w;
          }
        }
        if (tr) { GF_STAMP(0, i, 6); }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P is for the tensor core
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&bars->p_ready);
        if (tr) { GF_STAMP(0, i, 7); }
      }
      cnt = c0 + it.ntiles;
      // epilogue: O / l -> out; the two halves of a row add up their sums first
      if (ok) ok = mbar_wait(&bars->pv_done, (cnt - 1) & 1, abort_flag, err, 7);
      if (ok) {
        bars->row_max[mr & 1][half][r] = l;
        mbar_arrive(&bars->max_ready);
        ok = mbar_wait(&bars->max_ready, mr & 1, abort_flag, err, 11);
      }
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        l += bars->row_max[mr & 1][half ^ 1][r];
        ++mr;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* orow = out + ((size_t)(it.q_begin + it.r0 + r) * nh + it.head) * HD + half * (HD / 2);
        float o[HD / 2];
#pragma unroll
        for (int cc = 0; cc < HD / 2; cc += 32)
          tmem_ld32(tmem_o + lane_addr + half * (HD / 2) + cc,
                    *reinterpret_cast<float(*)[32]>(o + cc));
        tmem_ld_wait();
        // O is read: the next item's first P V may overwrite it while this one is stored
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&bars->o_free);
        if (live) {
#pragma unroll
          for (int k = 0; k < HD / 2; k += 8) {
            uint4 w;
            w.x = pack_bf16(o[k] * inv, o[k + 1] * inv);
            w.y = pack_bf16(o[k + 2] * inv, o[k + 3] * inv);
            w.z = pack_bf16(o[k + 4] * inv, o[k + 5] * inv);
            w.w = pack_bf16(o[k + 6] * inv, o[k + 7] * inv);
            *reinterpret_cast<uint4*>(orow + k) = w;
          }
        }
      }
      trace = false;
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (dbg && threadIdx.x == 0) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t) : : "memory");   // stays behind the barrier
    dbg[768 + cta_lin * 4 + 1] = (long long)t;
  }
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem),
                 "r"(TMEM_COLS)
                 : "memory");
  }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// rows x cols bf16 with `ld` elements between rows; box = box_rows x 64 channels, 128B swizzle
static bool make_map(CUtensorMap* map, const void* ptr, long long rows, int cols, long long ld,
                     int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
            estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_attn_tc_head_dim() { return HD; }

// q: T rows of q_row_stride elements whose first nh * HD hold the query heads; kpages / vpages:
// [num_pages, page_size, nkv, HD]; out [T, nh, HD].  Returns -6 for what it cannot serve (page
// sizes that are not a multiple of 8 or do not divide 128, unaligned pointers or strides).
GF_EXPORT int gf_attn_prefill_tc(const void* q, int q_row_stride, const void* kpages,
                                 const void* vpages, int num_pages, const int* block_table,
                                 int table_stride, const int* cu_seqlens_q, const int* kv_lens,
                                 void* out, int T, int B, int max_q_len, int nh, int nkv,
                                 int page_size, int window, float scale, int* err, void* dbg,
                                 void* stream) {
  if (B <= 0 || max_q_len <= 0 || T <= 0) return 0;
  if (nh % nkv || page_size % 8 || KT % page_size || page_size > KT) return -6;
  if (q_row_stride % 8 || ((uintptr_t)q & 15) || ((uintptr_t)kpages & 15) ||
      ((uintptr_t)vpages & 15) || ((uintptr_t)out & 15))
    return -6;
  const long long slots = (long long)num_pages * page_size;
  if (slots >= (1ll << 31) - page_size) return -6;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, q, T, nh * HD, q_row_stride, QT)) return -6;
  if (!make_map(&mk, kpages, slots, nkv * HD, (long long)nkv * HD, page_size)) return -6;
  if (!make_map(&mv, vpages, slots, nkv * HD, (long long)nkv * HD, page_size)) return -6;
  const size_t smem = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + P_BYTES +
                      sizeof(Barriers);
  static bool attr_done = false;
  if (!attr_done) {
    cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_done = true;
  }
  const int q_tiles = (max_q_len + QT - 1) / QT;
  const long long items = (long long)nh * q_tiles * B;
  if (items >= (1ll << 30)) return -6;
  int sms = 148, dev = 0, v = 0;
  if (cudaGetDevice(&dev) == cudaSuccess &&
      cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0)
    sms = v;
  dim3 grid((unsigned)(items < sms ? items : sms));
  return launch_kernel(attn_prefill_tc_kernel, grid, dim3(NTHREADS), smem, (cudaStream_t)stream,
                       mq, mk, mv, block_table, table_stride, cu_seqlens_q, kv_lens, (bf16*)out,
                       nh, nkv, page_size, window, scale * LOG2E, (int)slots, q_tiles, B, err,
                       (long long*)dbg);
}
