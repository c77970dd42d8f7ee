// Prefill attention on the 5th-generation tensor cores: varlen, causal (+ sliding window), GQA,
// over the paged cache.  Compiled for one head size (-DGF_HEAD_DIM = 64 or 128).
//
// One CTA owns 128 query rows of one head of one request.  Keys are visited in tiles of 128, and
// the tiles are dealt to two streams: stream 0 takes the item's tiles 0, 2, 4, ..., stream 1 the
// tiles 1, 3, 5, ...  Each stream has its own S, running maximum, sum and accumulator O_s, as if it
// were an attention over its own keys; at the end of the item the two are added up with the
// factors that bring them to a common maximum.  For a tile j of stream s:
//           S_s = Q K_j^T     tcgen05.mma, A = Q and B = K_j in shared memory (K-major, 128B
//                             swizzle, written by TMA), D = S_s in tensor memory (128 lanes x 128 fp32)
//           P_s = softmax     four warps a stream, one thread per query row: tcgen05.ld of its row
//                             of S_s, running maximum and sum in fp32, P_s rounded to bf16 and
//                             written back by tcgen05.st over the first 64 columns of S_s
//           O_s += P_s V_j    tcgen05.mma, A = P_s from tensor memory, B = V_j as stored
//                             ([key][channel], that is MN-major), D = O_s in tensor memory
// The tensor core alternates between the streams (P V and the next S of stream 0, then of stream
// 1), so that it works for one while the softmax warps of the other are busy: neither the tensor
// core nor the exponential unit waits for the other for long.  P never passes through shared
// memory, which halves the operand traffic of P V.
// An accumulator is rescaled in tensor memory only when a row's maximum has grown by more than
// 2^8 since the last rescale (the probabilities then stay below 2^8, well inside bf16 and fp32).
// K and V tiles come page by page through TMA: the cache of one layer is a 2-D tensor
// [token slots, kv_heads * HD]; a page is a box of page_size rows; pages past the request's end are
// loaded from out-of-range coordinates, which TMA fills with zeros.
//
// Warps: 0..3 = TMA loaders (K: 0-1, V: 2-3; every lane issues one box), 4 = tensor-memory
// allocation and MMA issue (5..7 only fill its warp group), 8..11 = softmax and epilogue of stream
// 0, 12..15 = of stream 1.  The kernel starts with 128 registers a thread; the first two warp
// groups give registers back and the softmax groups take them (setmaxnreg), so that a softmax
// thread holds its whole row of S.  The reference's prefill kernel is a 64x64 mma.sync flash loop
// with S, P and the row maximum held in bf16
// (ginfer/core/op/kernels/cuda/page_attn_kernel/flash_gqa_varlen_kernel.cu:420-512).
//
// What the structure answers to (measured on a B200; cycles per 128 x 128 tile): one query tile
// with S double buffered and P through shared memory, two threads a row: 2,750, bound by the
// chain load S - maximum - exponentials - store P of one tile at a time.  Two streams as above
// with a thread a row that reads S twice in chunks: the same 2,600 (the branch on "no key of
// this tile is masked" inside the loop over a chunk's keys had become the masked arithmetic for
// every key: four times slower, until it stood outside).  Packed fp32 arithmetic (fma.rn.f32x2,
// add.rn.f32x2, the three-input max): a lone warp on a scheduler spends 335 instead of 614 cycles
// on 32 scores.  The whole row in registers: 2,250.  The three waits of a group made by three
// lanes at once: 1,950 (a wait costs its thread 300 cycles while the tensor core reads its
// operands from shared memory, 60 otherwise).  The 16 products of a tile take 1,350 of them.
// Tried and not faster: a thread for each stream (the streams fall into step: both wait for the
// tensor core, then both for the exponentials), the same with turns handed over through barriers
// in shared memory (slower) or through a hardware barrier of the two warps (the same), the K and V
// waits moved to a softmax thread, a second warp that waits ahead and meets the issuing warp at
// a hardware barrier (4 % faster on long rows of tiles, 6 % slower on short ones), and a share of
// the exponentials by polynomial.  What a tile waits for now is the chain of one stream: softmax
// of a tile (2,150 cycles, 1,024 of them the exponential unit's), the wait of the issuing thread
// (300 to 500), the 16 products (1,350); two streams make two tiles in that time.
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
constexpr int NS = 2;                      // streams the key tiles are dealt to
constexpr int HALVES = HD / 64;            // 64-channel swizzle atoms per row
// Each stream has a ring of K tiles and a ring of V tiles of its own (so that every role meets
// every phase of the barriers it waits on): K_j is free as soon as S = Q K_j^T is computed, V_j
// once O += P V_j is complete.
constexpr int KS = 2;                              // K tiles a stream
constexpr int VS = HD == 128 ? 1 : 2;              // V tiles a stream
constexpr int K_STAGES = NS * KS, V_STAGES = NS * VS;
constexpr int NTHREADS = 512;              // four warp groups: loaders, MMA issue, softmax of stream 0, of stream 1
// Registers a thread: the kernel starts with 128 for all; the loader and MMA groups give registers
// back, the softmax groups take them, so that a softmax thread holds its whole row of S.
constexpr int REGS_SMALL = 64, REGS_SOFTMAX = 192;
static_assert(256 * REGS_SMALL + 256 * REGS_SOFTMAX <= 65536, "the register file of an SM");
constexpr uint32_t ATOM_BYTES = 128 * 64 * 2;            // a [128][64] bf16 tile: 16 KB
constexpr uint32_t Q_BYTES = HALVES * ATOM_BYTES;
constexpr uint32_t K_BYTES = HALVES * ATOM_BYTES;        // [128 keys][HD]
constexpr uint32_t V_BYTES = HALVES * ATOM_BYTES;
constexpr uint32_t TMEM_COLS = 512;     // S_0 / P_0: 0..127, S_1 / P_1: 128..255, O_0, O_1: 256..
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
// Bounded wait; gives up early when another role has raised the abort flag.  kFast: the waiter is
// on the critical path between the tensor core and the softmax warps and polls without sleeping
// for a good while.
template <bool kFast = false>
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
    if (spin > (kFast ? 4096u : 64u)) {
      if (*abort_flag) return false;
      __nanosleep(32);
    } else if (kFast && (spin & 255u) == 255u && *abort_flag) {
      return false;
    }
  }
  *abort_flag = 1;
  if (err) atomicExch(err, code);
  return false;
}
// The same for a whole warp, each lane with a barrier of its own (lanes without one pass
// `active` = false): returns when all of them are complete.  A wait costs its thread a few hundred
// cycles while the tensor core streams its operands out of shared memory, complete or not; three
// lanes make three waits in the time of one.
__device__ __forceinline__ bool mbar_wait_lanes(uint64_t* bar, uint32_t parity, bool active,
                                                volatile int* abort_flag, int* err, int code) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done = 1;
    if (active) {
      asm volatile(
          "{\n\t.reg .pred p;\n\t"
          "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
          "selp.u32 %0, 1, 0, p;\n\t}"
          : "=r"(done)
          : "r"(addr), "r"(parity)
          : "memory");
    }
    if (__all_sync(0xffffffffu, done != 0)) return true;
    active = active && !done;
    if (spin > 4096u) {
      if (*abort_flag) return false;
      __nanosleep(32);
    } else if ((spin & 255u) == 255u && *abort_flag) {
      return false;
    }
  }
  if ((threadIdx.x & 31) == 0) {
    *abort_flag = 1;
    if (err) atomicExch(err, code);
  }
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
// Shared-memory operand descriptors (sm_100 version, 128-byte swizzle), as a low word that holds
// the address (in 16-byte units; the issuing thread adds a tile's or a K step's offset to it with
// one 32-bit addition) and a high word that is the same for every operand of this kernel.
// K-major [rows][64]: rows 128 B apart, 8-row groups 1024 B apart.
// MN-major (V as stored: [key][channel]): a 128-byte row holds 64 channels of one key; 8 keys make
// a 1024-byte group (stride byte offset); the next 64 channels start one atom (16 KB) further on
// (leading byte offset).
constexpr uint32_t DESC_HI = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t saddr) {
  return ((saddr & 0x3FFFF) >> 4) | (1u << 16);
}
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t saddr) {
  return ((saddr & 0x3FFFF) >> 4) | ((ATOM_BYTES >> 4) << 16);
}
__device__ __forceinline__ uint64_t make_desc(uint32_t lo) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(DESC_HI));
  return d;
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
// The same with A taken from tensor memory: 128 lanes (rows) x 8 columns, two bf16 a column (the
// element with the lower K index in the low half).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t id,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(id), "r"(accumulate)
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
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
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
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),
      "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),
      "r"(v[15])
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
// Off unless the build asks for it: no share measured faster (a lone warp spends 335 cycles on 32
// scores with the unit, 450 with a quarter of them by polynomial).
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
// Two fp32 operations in one instruction (sm_100): the operands are pairs in 64-bit registers.
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

struct Barriers {
  uint64_t q_full;
  uint64_t q_empty;       // the item's last S product has read Q
  uint64_t k_full[K_STAGES];
  uint64_t k_empty[K_STAGES];
  uint64_t v_full[V_STAGES];
  uint64_t v_empty[V_STAGES];
  uint64_t s_full[NS];    // S of stream s is complete in tensor memory
  uint64_t p_ready[NS];   // P of stream s stands in tensor memory and O_s is rescaled (128 arrivals)
  uint64_t pv_done[NS];   // O_s += P_s V is complete
  uint64_t stat_ready;    // every row's (maximum, sum) of both streams is posted (256 arrivals)
  uint64_t o_free;        // the softmax warps have read an item's O_0 and O_1 out (256 arrivals)
  uint32_t tmem_base;
  int abort_flag;
  float stat_m[NS][QT];   // [stream][row]: the row's reference maximum and sum at the item's end
  float stat_l[NS][QT];
};

// One work item: 128 query rows of one head of one request, and the key tiles they see.
struct Item {
  int b, head, r0, rows, q_begin, pos0, key_lo, p_last, j0, ntiles, kvh;
};

__global__ void __launch_bounds__(NTHREADS, 1)
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
  Barriers* bars = reinterpret_cast<Barriers*>(v_s + V_STAGES * V_BYTES);
  volatile int* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // optional time stamps of the first CTA's first item (dbg: 8 slots per tile per role)
#ifdef GF_TRACE
  bool trace = dbg != nullptr && blockIdx.x == 0;
#else
  constexpr bool trace = false;     // the phase stamps are compiled in only with -DGF_TRACE
#endif
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
  // counts tiles and items for itself), so the loads and the first S products of the next item
  // overlap the last P V, the read-out and the stores of this one.
  const int items = nh * q_tiles * B;
  auto item_of = [&](int n, Item& it) -> int {   // 0: no more items, 1: it, 2: an empty item
    // (the roles copy the fields they use into variables of their own: the struct lies in local
    // memory, and a thread that issues products or copies would wait for loads from it)
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
  // stream s takes the item's key tiles s, s + 2, ...: how many
  auto tiles_of = [](int ntiles, int s) { return (ntiles - s + 1) >> 1; };

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
    for (int s = 0; s < NS; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_ready[s], QT);
      mbar_init(&bars->pv_done[s], 1);
    }
    mbar_init(&bars->stat_ready, NS * QT);
    mbar_init(&bars->o_free, NS * QT);
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
  // S (and, over its first 64 columns, P) of stream s at column 128 s; O of stream s behind them
  const uint32_t tmem_s = tmem, tmem_o = tmem + NS * KT;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SMALL));
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
    const int per_stream = is_v ? VS : KS;
    const uint32_t tile_bytes = is_v ? V_BYTES : K_BYTES;
    unsigned char* ring = is_v ? v_s : k_s;
    uint64_t* full = is_v ? bars->v_full : bars->k_full;
    uint64_t* empty = is_v ? bars->v_empty : bars->k_empty;
    const CUtensorMap* map = is_v ? &tmap_v : &tmap_k;
    const uint32_t my_bytes = (uint32_t)my_ops * (uint32_t)page_size * 128u;
    int cs[NS] = {0, 0};                                       // tiles of each stream so far
    int seq = 0;                                               // items so far
    bool go = true;
    Item it;
    for (int n = 0; go; ++n) {
      const int kind = item_of(n, it);
      if (kind == 0) break;
      if (kind == 2) continue;
      const int* tbl = block_table + (size_t)it.b * table_stride;
      const int ntiles = it.ntiles, j0 = it.j0, p_last = it.p_last, key_lo = it.key_lo,
                kv_col = it.kvh * HD;
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
        const int key0 = (j0 + i) * KT;
#pragma unroll
        for (int u = 0; u < MAX_OPS; ++u) {
          const int op = part + 2 * (lane + 32 * u);
          rows_next[u] = oob_row;
          if (op < ops && i < ntiles) {
            const int c = key0 + (op / HALVES) * page_size;    // first key of this page
            // pages past the request's last key (or wholly before the window) come from an
            // out-of-range row: TMA fills them with zeros
            if (c <= p_last && c + page_size > key_lo) {
              const int page = tbl[c / page_size];
              if (page >= 0) rows_next[u] = page * page_size;
            }
          }
        }
      };
      lookup(0);
      for (int i = 0; i < ntiles; ++i) {
        int rows_now[MAX_OPS];
#pragma unroll
        for (int u = 0; u < MAX_OPS; ++u) rows_now[u] = rows_next[u];
        int& cnt = (i & 1) ? cs[1] : cs[0];                    // tile i goes to stream i % 2
        const int st = (i & 1) * per_stream + cnt % per_stream;
        int ok = 1;
        if (lane == 0) {
          if (warp == 0) { GF_STAMP(2, i, 0); }
          ok = mbar_wait(&empty[st], ((cnt / per_stream) & 1) ^ 1, abort_flag, err, 1);
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
                        map, &full[st], kv_col + h * 64, rows_now[u]);
          }
        }
        if (warp == 0 && lane == 0) { GF_STAMP(2, i, 2); }
        ++cnt;
        lookup(i + 1);                                          // overlaps the next wait
      }
      ++seq;
#ifdef GF_TRACE
      trace = false;
#endif
    }
  } else if (warp < 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SMALL));
    // ------------------------------------------------------------------ MMA issuer
    // With t counting a stream's own tiles (stream s holds the item's tiles s, s + 2, ...), the
    // tensor core runs       O_0 += P_0 V_{2t},      S_0 = Q K_{2t+2}^T,
    //                        O_1 += P_1 V_{2t+1},    S_1 = Q K_{2t+3}^T
    // in this order, so that it works for one stream while the softmax warps of the other turn
    // their S into P.  The products of one thread complete in the order of issue, so the S
    // product that overwrites P_s (they share columns) runs behind the P V that reads it.
    if (warp == 4) {
      // The whole warp runs the loop; lane 0 issues the products, and lanes 0, 1 and 2 make the
      // three waits of a group (P, the V tile, the next K tile) at the same time.
      constexpr uint32_t id_qk = idesc(KT, false), id_pv = idesc(HD, true);
      const uint32_t q_desc = desc_lo_kmajor(smem_u32(q_s)), k_desc = desc_lo_kmajor(smem_u32(k_s)),
                     v_desc = desc_lo_mnmajor(smem_u32(v_s));
      int seq = 0;                                             // items so far
      int ck0 = 0, ck1 = 0, cv0 = 0, cv1 = 0;                  // S and P V products of each stream so far
      bool ok = true;
      Item it;
      for (int n = 0; ok; ++n) {
        const int kind = item_of(n, it);
        if (kind == 0) break;
        if (kind == 2) continue;
        const int ntiles = it.ntiles;
        // (every lane makes the waits of this loop; what they saw is made one answer for the warp,
        // since the waits by lanes below want every lane to take part)
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->q_full, (uint32_t)(seq & 1), abort_flag, err, 2));
        // S_s = Q K^T for the stream's next tile; `last`: the item's last tile
        auto issue_qk = [&](int s, bool last) {
          int& ck = s ? ck1 : ck0;
          const int st = s * KS + ck % KS;
          if (lane == 0) {
            const uint32_t kd = k_desc + st * (K_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < HD / 16; ++k) {
              const uint32_t off = ((k / 4) * ATOM_BYTES + (k % 4) * 32) >> 4;   // 16 channels = 32 bytes
              umma(tmem_s + KT * s, make_desc(q_desc + off), make_desc(kd + off), id_qk,
                   k > 0 ? 1u : 0u);
            }
            // (S complete means its K tile is free: the stream's softmax warps, who wait for S
            // anyway, say so to the loaders; a commit costs this thread as much as a product)
            umma_commit(&bars->s_full[s]);
            if (last) umma_commit(&bars->q_empty);  // Q has been read for the last time
          }
          ++ck;
        };
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          if (s >= ntiles || !ok) continue;
          const int ck = s ? ck1 : ck0;
          ok = __all_sync(0xffffffffu, mbar_wait<true>(&bars->k_full[s * KS + ck % KS], (ck / KS) & 1,
                                                    abort_flag, err, 3));
          if (!ok) continue;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_qk(s, s == ntiles - 1);
        }
        const int n0 = tiles_of(ntiles, 0);
        for (int t = 0; t < n0 && ok; ++t) {
#pragma unroll
          for (int s = 0; s < NS; ++s) {
            const int i = NS * t + s;
            if (i >= ntiles || !ok) continue;
            int& cv = s ? cv1 : cv0;
            const int ck = s ? ck1 : ck0;
            const int st = s * VS + cv % VS;
            if (lane == 0) { GF_STAMP(1, t, 4 * s); }
            // the item's first P V overwrites O: the item before must have been read out
            if (i == 0)
              ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_free, (uint32_t)(seq & 1) ^ 1u, abort_flag,
                                                     err, 14));
            if (lane == 0) { GF_STAMP(1, t, 4 * s + 1); }
            // lane 0: P of this tile; lane 1: its V tile; lane 2: the K tile of the next S product
            {
              uint64_t* bar = lane == 0   ? &bars->p_ready[s]
                              : lane == 1 ? &bars->v_full[st]
                                          : &bars->k_full[s * KS + ck % KS];
              const uint32_t par = lane == 0 ? (cv & 1) : lane == 1 ? ((cv / VS) & 1) : ((ck / KS) & 1);
              const bool active = lane < 2 || (lane == 2 && i + NS < ntiles);
              if (ok) ok = mbar_wait_lanes(bar, par, active, abort_flag, err, 4);
            }
            if (!ok) continue;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
              GF_STAMP(1, t, 4 * s + 2);
              const uint32_t vd = v_desc + st * (V_BYTES >> 4);
#pragma unroll
              for (int k = 0; k < KT / 16; ++k) {
                // 16 keys: 8 columns of P (two bf16 a column), 16 rows of V
                umma_ts(tmem_o + HD * s, tmem_s + KT * s + 8 * k,
                        make_desc(vd + ((k * 16 * 128) >> 4)), id_pv, (t > 0 || k > 0) ? 1u : 0u);
              }
            }
            if (i + NS < ntiles) issue_qk(s, i + NS == ntiles - 1);
            if (lane == 0) {
              umma_commit(&bars->v_empty[st]);        // the V tile may be overwritten
              if (i + NS >= ntiles) umma_commit(&bars->pv_done[s]);   // O_s holds all of the stream's tiles
              GF_STAMP(1, t, 4 * s + 3);
            }
            ++cv;
          }
        }
        ++seq;
#ifdef GF_TRACE
        trace = false;
#endif
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_SOFTMAX));
    // ------------------------------------------------------------------ softmax + epilogue
    // Eight warps: four for each stream, one thread per query row with all 128 keys of a tile, so
    // that no two threads share a row while the tiles are visited, and the two groups are at
    // different points of their tiles: one group's exponentials run beside the other's loads,
    // maxima and stores.  Each stream keeps a maximum, a sum and an accumulator O_s of its own;
    // at the end of the item the two are added up with the factors that bring them to a common
    // maximum.  A thread holds its whole row of S in registers (these warp groups have taken the
    // registers the others gave back) and writes P as bf16 over the first columns of S; the
    // tensor core takes P from there.
    const int qd = warp & 3;                                   // TMEM lane quarter of this warp
    const int s = (warp - 8) >> 2;                             // stream of this warp
    const int r = qd * 32 + lane;                              // query row of this thread
    const uint32_t lane_addr = (uint32_t)(qd * 32) << 16;
    const uint32_t my_s = tmem_s + KT * s + lane_addr, my_o = tmem_o + HD * s + lane_addr;
    int cnt = 0, seq = 0;                                      // tiles of this stream, items so far
    int had = 0;                                               // items in which this stream had tiles
    bool ok = true;
    Item it;
    for (int n = 0; ok; ++n) {
      const int kind = item_of(n, it);
      if (kind == 0) break;
      if (kind == 2) continue;
      const int ntiles = it.ntiles, rows = it.rows, j0 = it.j0, row0 = it.q_begin + it.r0,
                head = it.head, pos00 = it.pos0 + it.r0;      // position of the item's first row
      const int mine = tiles_of(ntiles, s);
      const int p = pos00 + r;                                 // this row's position
      const bool live = r < rows;
      const int lo = window > 0 ? max(0, p - window + 1) : 0;
      const int wp0 = pos00 + qd * 32;                         // position of the warp's first row
      const bool tr = r == 0;
      float m_used = -INFINITY;        // the maximum the accumulated P and l are scaled by
      float l = 0.f;                   // the row sum
      for (int t = 0; t < mine; ++t, ++cnt) {
        const int i = 2 * t + s;
        if (tr) { GF_STAMP(0, i, 0); }
        ok = mbar_wait<true>(&bars->s_full[s], cnt & 1, abort_flag, err, 5);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (tr) { GF_STAMP(0, i, 1); }
        if (r == 0) mbar_arrive(&bars->k_empty[s * KS + cnt % KS]);   // S is computed: its K tile is free
        const int col0 = (j0 + i) * KT;                        // first key of the tile
        // every row of this warp sees all of the tile's keys: no comparisons
        const bool interior = col0 + KT - 1 <= wp0 && qd * 32 + 32 <= rows &&
                              (window <= 0 || col0 >= wp0 + 31 - window + 1);
        // ---- the whole row of S into registers
        float v[KT];
#pragma unroll
        for (int cc = 0; cc < KT / 32; ++cc)
          tmem_ld32(my_s + 32 * cc, *reinterpret_cast<float(*)[32]>(v + 32 * cc));
        tmem_ld_wait();
        if (!interior) {
#pragma unroll
          for (int k = 0; k < KT; ++k) {
            const int key = col0 + k;
            v[k] = (live && key >= lo && key <= p) ? v[k] : -INFINITY;
          }
        }
        // ---- the row's maximum (eight running maxima instead of one chain)
        float mx8[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) mx8[j] = -INFINITY;
#pragma unroll
        for (int k = 0; k < KT; k += 2) mx8[(k >> 1) & 7] = max3(mx8[(k >> 1) & 7], v[k], v[k + 1]);
        const float mx = fmaxf(max3(mx8[0], mx8[1], mx8[2]), max3(mx8[3], mx8[4], max3(mx8[5], mx8[6], mx8[7]))) *
                         scale_log2;                            // scale > 0
        if (tr) { GF_STAMP(0, i, 2); }
        // lazy rescale: keep the old reference maximum unless the row's maximum outgrew it
        float m_new = m_used;
        if (mx > m_used + kRescaleStep || m_used == -INFINITY) m_new = fmaxf(m_used, mx);
        const float corr = (m_new == m_used) ? 1.f
                           : (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new));
        const float msub = m_new == -INFINITY ? 0.f : m_new;
        // S of this tile is complete, so the stream's P V of the tile before (issued ahead of
        // it) is too: O_s is at rest and may be rescaled (the stream's first P V overwrites O_s)
        if (t > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll 1
          for (int cc = 0; cc < HD; cc += 16) {
            float o[16];
            tmem_ld16(my_o + cc, o);
            tmem_ld_wait();
            uint32_t ob[16];
#pragma unroll
            for (int k = 0; k < 16; ++k) ob[k] = __float_as_uint(o[k] * corr);
            tmem_st16(my_o + cc, ob);
          }
        }
        // ---- probabilities (bf16, over the first 64 columns of S) and the row sum
        uint64_t sum2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};       // four partial sums
        const uint64_t scale2 = pack2(scale_log2, scale_log2), msub2 = pack2(-msub, -msub);
#pragma unroll
        for (int cc = 0; cc < KT / 32; ++cc) {
          uint32_t w[16];
#pragma unroll
          for (int k = 0; k < 32; k += 2) {
            float a0, a1, e0, e1;
            unpack2(fma2(pack2(v[32 * cc + k], v[32 * cc + k + 1]), scale2, msub2), a0, a1);
            if (GF_POLY_EXP_EVERY > 0 &&
                (k / 2) % (GF_POLY_EXP_EVERY > 0 ? GF_POLY_EXP_EVERY : 1) == GF_POLY_EXP_EVERY - 1) {
              e0 = poly_exp2(a0);             // clamps at -125: a masked key gives 2^-125 = nothing
              e1 = poly_exp2(a1);
            } else {
              e0 = fast_exp2(a0);
              e1 = fast_exp2(a1);
            }
            sum2[(k >> 1) & 1] = add2(sum2[(k >> 1) & 1], pack2(e0, e1));
            w[k / 2] = pack_bf16(e0, e1);
          }
          tmem_st16(my_s + 16 * cc, w);
        }
        {
          float s0, s1, s2, s3;
          unpack2(sum2[0], s0, s1);
          unpack2(sum2[1], s2, s3);
          l = l * corr + ((s0 + s1) + (s2 + s3));
        }
        m_used = m_new;
        if (tr) { GF_STAMP(0, i, 3); }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(&bars->p_ready[s]);
        if (tr) { GF_STAMP(0, i, 4); }
      }
      if (!ok) break;
      // ---- end of the item: the stream's last P V, then both streams' (maximum, sum) of the row
      if (mine > 0) {
        ok = mbar_wait(&bars->pv_done[s], had & 1, abort_flag, err, 7);
        ++had;
      }
      if (!ok) break;
      // (the item before has been read out by every thread, so its figures are not needed any more)
      if (seq > 0) ok = mbar_wait(&bars->o_free, (uint32_t)(seq - 1) & 1u, abort_flag, err, 15);
      if (!ok) break;
      bars->stat_m[s][r] = m_used;
      bars->stat_l[s][r] = l;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&bars->stat_ready);
      ok = mbar_wait(&bars->stat_ready, seq & 1, abort_flag, err, 11);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float m_o = bars->stat_m[s ^ 1][r], l_o = bars->stat_l[s ^ 1][r];
      const float m_all = fmaxf(m_used, m_o);
      const float f_me = m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_all);
      const float f_o = m_o == -INFINITY ? 0.f : fast_exp2(m_o - m_all);
      const float l_all = l * f_me + l_o * f_o;
      const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
      // this stream writes channels s * HD / 2 .. of the row: from O_0 and (if stream 1 had a
      // tile at all) O_1, each with its stream's factor
      const float f0 = (s == 0 ? f_me : f_o) * inv, f1 = (s == 0 ? f_o : f_me) * inv;
      const bool two = ntiles > 1;
      const uint32_t o0 = tmem_o + lane_addr + s * (HD / 2), o1 = o0 + HD;
      bf16* orow = out + ((size_t)(row0 + r) * nh + head) * HD + s * (HD / 2);
#pragma unroll 1
      for (int cc = 0; cc < HD / 2; cc += 16) {
        float a[16], b[16];
        tmem_ld16(o0 + cc, a);
        if (two) tmem_ld16(o1 + cc, b);
        tmem_ld_wait();
        if (cc + 16 >= HD / 2) {
          // O is read: the next item's first P V may overwrite it while this one is stored
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          mbar_arrive(&bars->o_free);
        }
        if (live) {
#pragma unroll
          for (int k = 0; k < 16; ++k) a[k] = two ? fmaf(b[k], f1, a[k] * f0) : a[k] * f0;
#pragma unroll
          for (int k = 0; k < 16; k += 8) {
            uint4 w;
            w.x = pack_bf16(a[k], a[k + 1]);
            w.y = pack_bf16(a[k + 2], a[k + 3]);
            w.z = pack_bf16(a[k + 4], a[k + 5]);
            w.w = pack_bf16(a[k + 6], a[k + 7]);
            *reinterpret_cast<uint4*>(orow + cc + k) = w;
          }
        }
      }
      ++seq;
#ifdef GF_TRACE
      trace = false;
#endif
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
  const size_t smem = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + sizeof(Barriers);
  static OncePerDevice attrs;
  if (int rc = attrs.run([&] {
        return cudaFuncSetAttribute(attn_prefill_tc_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      }))
    return rc;
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
