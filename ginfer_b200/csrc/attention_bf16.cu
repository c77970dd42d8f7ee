// bf16 grouped-query attention over the paged cache for the serving path, compiled for one head
// size (-DGF_HEAD_DIM=<multiple of 16, at most 256>).
//
//  * gf_attn_decode_tma: one query token per request, for head sizes that are a multiple of 64 and
//    page sizes that fit the 64-key tile: tiles by TMA through a loader warp, query heads as the 8
//    columns of the tensor-core tiles (described where the kernel stands, further down).
//  * gf_attn_decode: the same for every head size and page size.  One CTA per (request, kv head,
//    split of the keys, chunk of 16 query heads): the query heads of a group share every K/V byte that is
//    loaded (the reference's decode kernel reads K/V once per query head:
//    ginfer/core/op/kernels/cuda/page_attn_kernel/flash_gqa_varlen_decode_kvcache.cu:272-335).
//    Splits write fp32 partial results (running maximum, sum, unnormalised output) to scratch
//    memory; the CTA that finishes a (request, kv head) last merges them (a second kernel does it
//    when there are more such groups than counters).
//  * gf_attn_prefill: any number of query tokens per request (portions of prompts, and single
//    tokens beside them).  One CTA per (128 query rows of one head; 64 for head sizes above 128);
//    keys are visited in tiles of 64 through the block table.
//
// Both use mma.sync.m16n8k16 (bf16 in, fp32 accumulate) with operands staged in shared memory by
// cp.async and read by ldmatrix.  Scores, the running maximum, the sum and the output accumulator
// are fp32 (the reference keeps S, P, the maximum and O in bf16:
// flash_gqa_varlen_kernel.cu:169-172,220-257); P is rounded to bf16 for the P*V product.
// Visibility: the query at position p sees key c iff c <= p and (window == 0 or p - c < window).
#include <mutex>

#include "attention_mma.cuh"
#include "tc_common.cuh"

namespace gf {

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem(const float* local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)),
               "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

// The cluster's CTAs combine their partial results: every CTA a share of the output channels,
// over all peers' partials, read through distributed shared memory in split order.
template <int MAXC>
__device__ __forceinline__ void cluster_merge(float* cpart, float* cpart_m, float* cpart_l,
                                              float* cw, float* cinv, bf16* __restrict__ out,
                                              int nrows, int splits, int split, int row, int nh,
                                              int h0, bool active = true, float* part_o = nullptr,
                                              float* part_ml = nullptr, int parts = 1) {
  // Loads from the peers are issued eight at a time without branches (the peer index is
  // clamped, a clamped load's weight is zero); the additions stay in split order.
  // (`active` false: a thread beyond the NTHREADS that work here; it only joins the barrier)
  if (threadIdx.x < nrows) {
    const int r = threadIdx.x;
    float mp[MAXC], lp[MAXC];
#pragma unroll
    for (int p = 0; p < MAXC; ++p) {
      const uint32_t peer = (uint32_t)min(p, splits - 1);
      mp[p] = ld_dsmem(cpart_m + r, peer);
      lp[p] = ld_dsmem(cpart_l + r, peer);
    }
    float mm = -INFINITY;
#pragma unroll
    for (int p = 0; p < MAXC; ++p)
      if (p < splits) mm = fmaxf(mm, mp[p]);
    float lsum = 0.f;
#pragma unroll
    for (int p = 0; p < MAXC; ++p) {
      const float wgt = (p < splits && mp[p] != -INFINITY) ? exp2f(mp[p] - mm) : 0.f;
      cw[r * 16 + p] = wgt;
      lsum += wgt * lp[p];
    }
    cinv[r] = lsum > 0.f ? 1.f / lsum : 0.f;
    // part_o / part_ml: this cluster holds only a part of the request's keys; it leaves its
    // unnormalised result with the maximum and the sum for the kernel that merges the parts
    // (both pointers stand at this cluster's part of its first head; a head has `parts` parts)
    if (part_ml && split == 0) {
      part_ml[(size_t)r * parts * 2] = mm;
      part_ml[(size_t)r * parts * 2 + 1] = lsum;
    }
  }
  __syncthreads();
  const int total = nrows * HD, share = (total + splits - 1) / splits;
  const int i0 = split * share, i1 = min(total, i0 + share);
  for (int i = i0 + threadIdx.x; i < i1 && active; i += NTHREADS) {
    const int r = i / HD, d = i - r * HD;
    float v[MAXC];
#pragma unroll
    for (int p = 0; p < MAXC; ++p) v[p] = ld_dsmem(cpart + i, (uint32_t)min(p, splits - 1));
    float acc = 0.f;
#pragma unroll
    for (int p = 0; p < MAXC; ++p) acc += p < splits ? cw[r * 16 + p] * v[p] : 0.f;
    if (part_o) part_o[(size_t)r * parts * HD + d] = acc;
    else out[((size_t)row * nh + h0 + r) * HD + d] = __float2bfloat16_rn(acc * cinv[r]);
  }
}

// ================================================================================== decode
// grid (splits, nkv * head_chunks, B); 4 warps, warp w owns keys [16w, 16w + 16) of every tile.
// Partials: po [B, nh, splits, HD] fp32 unnormalised, pml [B, nh, splits, 2] = (max in log2 units,
// sum).  With one split the normalised bf16 result goes straight to `out`.
constexpr int DEC_STAGES = 3;
// With `fused` set, q and the new token's k arrive unrotated in the q/k/v row: the kernel rotates
// q by the angles of the token's position (table row: cos | sin, `rot` channels wide) and the
// split that holds the token's position rotates k, and writes k and v to their cache slot, before
// it reads that range of keys.  One launch less than rotating and writing in a kernel before.
struct RopeArgs {
  const float* table;          // [positions][rot] or null (nothing is rotated)
  int rot;
  int fused;                   // 0: q is rotated and the cache written already
  int write_kv;                // 0: the cache is another layer's to write
};
constexpr int kMaxTableCopy = 4096;   // block-table entries a CTA copies to shared memory at most
constexpr int kMaxDevicesTracked = 64;        // devices whose per-device set-up is remembered
constexpr int kMaxDecodeGroups = 1 << 16;     // (request, kv head, head chunk) triples with a counter
__device__ unsigned int g_decode_done[kMaxDecodeGroups];

__global__ void __launch_bounds__(NTHREADS)
attn_decode_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ kpages,
                   const bf16* __restrict__ vpages, const int* __restrict__ block_table,
                   int table_stride, const int* __restrict__ cu_seqlens_q,
                   const int* __restrict__ positions, bf16* __restrict__ out,
                   float* __restrict__ po, float* __restrict__ pml, int nh, int nkv,
                   int page_size, int window, float scale_log2, int splits, int fused_merge,
                   int tbl_off, int tbl_cap, const RopeArgs rope) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ bool last_split;
  bf16* ks = reinterpret_cast<bf16*>(smem_raw);                 // [STAGES][KT][ROW]
  bf16* vs = ks + DEC_STAGES * KT * ROW;                        // [STAGES][KT][ROW]
  const int split = blockIdx.x, b = blockIdx.z;
  const int G = nh / nkv;
  const int chunks = (G + 15) / 16;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;
  const int h0 = kvh * G + chunk * 16;                          // first query head of this CTA
  const int nrows = min(16, G - chunk * 16);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  pdl_trigger();
  // When this kernel itself writes the new token's k and v, the keys it reads from the cache are
  // all from earlier steps (the new token's come through shared memory): the first tiles are
  // fetched before the wait for the kernel in front (the q/k/v product), whose tail they overlap.
  const bool late_wait = rope.fused && rope.write_kv;
  if (!late_wait) pdl_wait();
  const int row = cu_seqlens_q ? cu_seqlens_q[b] : b;         // null: request b is row b
  const int p = positions[row];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int nkeys = p - lo + 1;
  int per = (nkeys + splits - 1) / splits;
  per = (per + KT - 1) / KT * KT;
  const int begin = lo + split * per;
  const int end = min(p + 1, begin + per);
  const int* tbl = block_table + (size_t)b * table_stride;
  const size_t tok_stride = (size_t)nkv * HD;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

  float o[HD / 8][4];
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const int lo2[2] = {begin, begin}, hi2[2] = {end - 1, end - 1};

  const int ntiles = begin < end ? (end - begin + KT - 1) / KT : 0;
  // this split's block-table entries -> shared memory
  int lp_base = 0;
  if (ntiles > 0) {
    const int lp0 = begin / page_size, nlp = (end - 1) / page_size - lp0 + 1;
    if (nlp <= tbl_cap) {
      int* stbl = reinterpret_cast<int*>(smem_raw + tbl_off);
      for (int i = threadIdx.x; i < nlp; i += NTHREADS) stbl[i] = tbl[lp0 + i];
      __syncthreads();
      tbl = stbl;
      lp_base = lp0;
    }
  }
  for (int s = 0; s < DEC_STAGES - 1; ++s) {
    if (s < ntiles)
      load_kv_tiles(ks + s * KT * ROW, vs + s * KT * ROW, kpages, vpages, tbl, lp_base,
                    begin + s * KT, begin, end, page_size, page_shift, tok_stride, kvh, threadIdx.x);
    cp_async_commit();
  }
  if (late_wait) pdl_wait();     // everything above read only what earlier steps and the host wrote
  // query fragments: rows are the heads h0 + g and h0 + g + 8; straight from global memory, or
  // (fused rotation) rotated into shared memory first
  uint32_t qf[KCH][4];
  const bf16* qrow = q + (size_t)row * q_row_stride + (size_t)h0 * HD;
  const int q_ld = HD;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw + tbl_off + (size_t)tbl_cap * sizeof(int));
  bf16* knew = qs + 16 * HD;   // [HD], then v [HD]
  bf16* vnew = knew + HD;
  bool patch = false;          // the last tile of this CTA gets the new token's k and v from here
  if (rope.fused && begin < end) {
    const bf16* base = q + (size_t)row * q_row_stride;
    const int half = rope.rot >> 1, tail = HD - rope.rot;
    const float* cs = rope.table ? rope.table + (size_t)p * rope.rot : nullptr;
    for (int i = threadIdx.x; i < nrows * half; i += NTHREADS) {
      const int r = i / half, j = i - r * half;
      const float a = __bfloat162float(qrow[r * HD + j]);
      const float bb = __bfloat162float(qrow[r * HD + j + half]);
      const float c = cs[j], sn = cs[half + j];
      qs[r * HD + j] = __float2bfloat16_rn(a * c - bb * sn);
      qs[r * HD + j + half] = __float2bfloat16_rn(a * sn + bb * c);
    }
    for (int i = threadIdx.x; i < nrows * tail; i += NTHREADS) {
      const int r = i / tail, j = rope.rot + (i - r * tail);
      qs[r * HD + j] = qrow[r * HD + j];
    }
    if (rope.write_kv && p >= begin && p < end) {
      // This split holds the new token.  Its k (rotated) and v are kept in shared memory and put
      // into the tile of keys once that has landed, so that no CTA depends on when another one's
      // write reaches memory; the CTA of the first head chunk also writes them to the cache slot.
      patch = true;
      const int lp = p / page_size;
      const size_t slot = (size_t)block_table[(size_t)b * table_stride + lp] * page_size +
                          (size_t)(p - lp * page_size);
      bf16* kd = const_cast<bf16*>(kpages) + slot * ((size_t)nkv * HD) + (size_t)kvh * HD;
      bf16* vd = const_cast<bf16*>(vpages) + slot * ((size_t)nkv * HD) + (size_t)kvh * HD;
      const bf16* kn = base + (size_t)(nh + kvh) * HD;
      const bf16* vn = base + (size_t)(nh + nkv + kvh) * HD;
      const bool store = chunk == 0;
      for (int j = threadIdx.x; j < half; j += NTHREADS) {
        const float a = __bfloat162float(kn[j]), bb = __bfloat162float(kn[j + half]);
        const float c = cs[j], sn = cs[half + j];
        const bf16 lo_v = __float2bfloat16_rn(a * c - bb * sn);
        const bf16 hi_v = __float2bfloat16_rn(a * sn + bb * c);
        knew[j] = lo_v, knew[j + half] = hi_v;
        if (store) kd[j] = lo_v, kd[j + half] = hi_v;
      }
      for (int j = rope.rot + threadIdx.x; j < HD; j += NTHREADS) {
        knew[j] = kn[j];
        if (store) kd[j] = kn[j];
      }
      for (int j = threadIdx.x; j < HD; j += NTHREADS) {
        vnew[j] = vn[j];
        if (store) vd[j] = vn[j];
      }
    }
    __syncthreads();             // q, and the new k and v, are in shared memory
    qrow = qs;
  }
  {
#pragma unroll
    for (int kc = 0; kc < KCH; ++kc) {
      const int d = kc * 16 + 2 * t;
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(qrow + (size_t)g * q_ld + d);
      const uint32_t* r1 = reinterpret_cast<const uint32_t*>(qrow + (size_t)(g + 8) * q_ld + d);
      qf[kc][0] = g < nrows ? r0[0] : 0u;
      qf[kc][1] = g + 8 < nrows ? r1[0] : 0u;
      qf[kc][2] = g < nrows ? r0[4] : 0u;
      qf[kc][3] = g + 8 < nrows ? r1[4] : 0u;
    }
  }
  for (int it = 0; it < ntiles; ++it) {
    cp_async_wait<DEC_STAGES - 2>();
    __syncthreads();
    if (patch && it == ntiles - 1) {
      const int st = it % DEC_STAGES, rp = p - (begin + it * KT);
      for (int j = threadIdx.x; j < HD; j += NTHREADS) {
        ks[(st * KT + rp) * ROW + j] = knew[j];
        vs[(st * KT + rp) * ROW + j] = vnew[j];
      }
      __syncthreads();
    }
    const int nxt = it + DEC_STAGES - 1;
    if (nxt < ntiles) {
      const int st = nxt % DEC_STAGES;
      load_kv_tiles(ks + st * KT * ROW, vs + st * KT * ROW, kpages, vpages, tbl, lp_base,
                    begin + nxt * KT, begin, end, page_size, page_shift, tok_stride, kvh, threadIdx.x);
    }
    cp_async_commit();
    const int st = it % DEC_STAGES;
    const int col0 = begin + it * KT + warp * 16;
    if (col0 < end) {
      float s[2][4] = {};
      qk_tile<2>(s, qf, ks + st * KT * ROW, warp * 16, lane);
      if (col0 + 16 <= end)
        softmax_update<2, false>(s, o, m, l, col0, lo2, hi2, scale_log2, lane);
      else
        softmax_update<2, true>(s, o, m, l, col0, lo2, hi2, scale_log2, lane);
      pv_tile<2>(o, s, vs + st * KT * ROW, warp * 16, lane);
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // merge the four warps through shared memory (reusing the tile buffers)
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
  // (rows 8 floats apart in banks: the 8-byte stores of a half-warp then hit every bank once)
  constexpr int SOP = HD + 8;
  float* so = reinterpret_cast<float*>(smem_raw);               // [4][16][SOP]
  float* sm = so + 4 * 16 * SOP;                                // [4][16]
  float* sl = sm + 4 * 16;                                      // [4][16]
  float* cpart = sl + 4 * 16;                                   // [16][HD]: the CTA's partial
  float* cpart_m = cpart + 16 * HD;                             // [16]
  float* cpart_l = cpart_m + 16;                                // [16]
  float* ww = cpart_l + 16;                                     // [4][16]: a warp's weight in a row
#pragma unroll
  for (int n = 0; n < HD / 8; ++n) {
    float* base = so + (warp * 16) * SOP + n * 8 + 2 * t;
    *reinterpret_cast<float2*>(base + g * SOP) = make_float2(o[n][0], o[n][1]);
    *reinterpret_cast<float2*>(base + (g + 8) * SOP) = make_float2(o[n][2], o[n][3]);
  }
  if (t == 0) {
    sm[warp * 16 + g] = m[0];
    sm[warp * 16 + g + 8] = m[1];
    sl[warp * 16 + g] = l[0];
    sl[warp * 16 + g + 8] = l[1];
  }
  __syncthreads();
  if (threadIdx.x < 64) {
    const int r = threadIdx.x & 15;
    const float mm = fmaxf(fmaxf(sm[r], sm[16 + r]), fmaxf(sm[32 + r], sm[48 + r]));
    ww[threadIdx.x] = mm == -INFINITY ? 0.f : exp2f(sm[threadIdx.x] - mm);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * HD; i += NTHREADS) {
    const int r = i / HD, d = i - r * HD;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) acc += ww[w * 16 + r] * so[(w * 16 + r) * SOP + d];
    float mm = -INFINITY, lsum = 0.f;
    if (d == 0 || splits == 1) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mm = fmaxf(mm, sm[w * 16 + r]);
        lsum += ww[w * 16 + r] * sl[w * 16 + r];
      }
    }
    const int head = h0 + r;
    if (splits == 1) {
      out[((size_t)row * nh + head) * HD + d] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    } else if (fused_merge == 2) {
      cpart[i] = acc;                                   // this CTA's partial stays in shared memory
      if (d == 0) {
        cpart_m[r] = mm;
        cpart_l[r] = lsum;
      }
    } else {
      const size_t pi = ((size_t)b * nh + head) * splits + split;
      po[pi * HD + d] = acc;
      if (d == 0) {
        pml[pi * 2] = mm;
        pml[pi * 2 + 1] = lsum;
      }
    }
  }
  if (fused_merge == 2 && splits > 1) {
    // The splits of a (request, kv head) form a thread-block cluster: after a cluster barrier every
    // CTA combines a share of the output channels over all peers' partials, read through
    // distributed shared memory in split order.  No scratch in global memory, no atomics.
    cluster_sync_all();
    float* cw = cpart_l + 16;                           // [16 rows][16 splits] weights
    float* cinv = cw + 256;                             // [16]
    if (splits <= 8)
      cluster_merge<8>(cpart, cpart_m, cpart_l, cw, cinv, out, nrows, splits, split, row, nh, h0);
    else
      cluster_merge<16>(cpart, cpart_m, cpart_l, cw, cinv, out, nrows, splits, split, row, nh, h0);
    cluster_sync_all();                                 // nobody leaves while a peer reads it
    return;
  }
  if (splits == 1 || !fused_merge) return;
  // the CTA that finishes this (request, kv head, chunk) last merges the splits' partial results
  __threadfence();
  __syncthreads();
  const unsigned int group = (unsigned int)b * gridDim.y + blockIdx.y;
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&g_decode_done[group], 1u);
    last_split = done == (unsigned int)splits - 1;
    if (last_split) g_decode_done[group] = 0;                   // ready for the next launch
  }
  __syncthreads();
  if (!last_split) return;
  __threadfence();
  // weights of the splits first (through shared memory), then every thread adds up its channels
  // with independent loads; splits past the request's keys hold nothing and are passed over
  const int used = min(splits, per > 0 ? (nkeys + per - 1) / per : 0);
  float* w = reinterpret_cast<float*>(smem_raw);                 // [16][used]: weight of a split
  float* linv = w + 16 * used;                                   // [16]: 1 / total sum
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * used; i += NTHREADS) {
    const int r = i / used, s2 = i - r * used;
    const size_t base = ((size_t)b * nh + h0 + r) * splits;
    w[r * used + s2] = __ldcg(pml + (base + s2) * 2);            // the split's maximum for now
  }
  __syncthreads();
  if (threadIdx.x < nrows) {
    const int r = threadIdx.x;
    const size_t base = ((size_t)b * nh + h0 + r) * splits;
    float mm = -INFINITY;
    for (int s2 = 0; s2 < used; ++s2) mm = fmaxf(mm, w[r * used + s2]);
    float lsum = 0.f;
    for (int s2 = 0; s2 < used; ++s2) {
      const float ms = w[r * used + s2];
      const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - mm);
      w[r * used + s2] = wgt;
      lsum += wgt * __ldcg(pml + (base + s2) * 2 + 1);
    }
    linv[r] = lsum > 0.f ? 1.f / lsum : 0.f;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * HD; i += NTHREADS) {
    const int r = i / HD, d = i - r * HD;
    const float* p = po + ((size_t)b * nh + h0 + r) * splits * HD + d;
    float acc = 0.f;
#pragma unroll 4
    for (int s2 = 0; s2 < used; ++s2) acc += w[r * used + s2] * __ldcg(p + (size_t)s2 * HD);
    out[((size_t)row * nh + h0 + r) * HD + d] = __float2bfloat16_rn(acc * linv[r]);
  }
}

#if GF_HEAD_DIM % 64 == 0
// ================================================================== decode, tiles by TMA
// The same split-KV decode for head sizes that are a multiple of 64 and page sizes that divide (or
// are a multiple of) the 64-key tile, built for bandwidth: at many requests or long contexts the
// kernel above spends its time on instructions (about 750 per warp and 16 keys: 16-byte copies
// with their page look-ups, and tensor-core tiles that are 16 query heads wide although a group
// has at most 8).  Here
//  * K and V tiles come by TMA, one box per page and 64-channel half, issued by the lanes of
//    a fifth warp that does nothing else (issuing a tile's 16 boxes takes longer than the
//    arithmetic on the tile), into 128-byte-swizzled rows (no padding: 32 KB a stage at head
//    size 128); a page past the request's keys is loaded from a row outside the tensor, which
//    TMA fills with zeros;
//  * the roles in the tensor-core tiles are swapped: keys (or channels) are the 16 rows and the
//    group's query heads the 8 columns.  S^T = K Q^T takes HD/16 instructions per 16 keys and
//    O^T += V^T P^T another HD/16 (half of what 16-row head tiles take), P^T reaches its operand
//    layout by two movmatrix transposes, and the accumulator is HD/4 registers instead of HD/2.
// Groups of more than 8 query heads take several CTAs (chunks of 8).  The splits merge inside a
// thread-block cluster as above.  Arithmetic is the same (fp32 scores, maxima, sums, accumulator).
constexpr int HALVES = HD / 64;
constexpr int TMAX_STAGES = 6;                         // ring depth: 2 .. 6, chosen per launch
constexpr uint32_t HALF_BYTES = KT * 128;                // [64 keys][64 channels] of bf16
constexpr uint32_t TILE_BYTES = HALVES * HALF_BYTES;     // K (or V) of a stage
constexpr uint32_t STAGE_BYTES = 2 * TILE_BYTES;
constexpr int kMaxTableCopyTma = 2048;

__device__ __forceinline__ uint32_t movmatrix_t(uint32_t v) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(v));
  return d;
}
// byte offset, inside a K or V tile, of the 8 channels from `ch` (a multiple of 8) of key row `key`
__device__ __forceinline__ uint32_t swz(int key, int ch) {
  return (uint32_t)(ch >> 6) * HALF_BYTES + (uint32_t)key * 128u +
         (uint32_t)((((ch >> 3) & 7) ^ (key & 7)) << 4);
}

constexpr int TMA_THREADS = NTHREADS + 32;               // four consumer warps and the loader
__device__ __forceinline__ void consumer_sync() {        // the four consumer warps only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

__global__ void __launch_bounds__(TMA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap kmap,
                       const __grid_constant__ CUtensorMap vmap, const bf16* __restrict__ q,
                       int q_row_stride, bf16* __restrict__ kpages, bf16* __restrict__ vpages,
                       const int* __restrict__ block_table, int table_stride,
                       const int* __restrict__ cu_seqlens_q, const int* __restrict__ positions,
                       bf16* __restrict__ out, int nh, int nkv, int page_size, int window,
                       float scale_log2, int splits, int oob_row, int tbl_cap, int nst,
                       int* err, const RopeArgs rope, int parts, float* __restrict__ po,
                       float* __restrict__ pml) {
  // No static shared memory in this kernel: the dynamic part then starts at the aligned base,
  // which the swizzled tiles need (checked below: a misaligned base ends the CTA with code 5).
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* ring = smem_raw;                               // [nst][K tile | V tile]
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)nst * STAGE_BYTES);
  uint64_t* empty = full + TMAX_STAGES;
  uint64_t* patched = full + 2 * TMAX_STAGES;                   // the new key and value are in their tile
  int* stbl = reinterpret_cast<int*>(full + 2 * TMAX_STAGES + 1);
  bf16* qs = reinterpret_cast<bf16*>(stbl + tbl_cap);           // [8][HD] rotated q, then new k, v
  bf16* knew = qs + 8 * HD;
  bf16* vnew = knew + HD;
  // grid z = request * parts + part: with `parts` > 1 several clusters share a request's keys,
  // each leaves an unnormalised result in po / pml, and attn_decode_merge_kernel adds them up
  const int split = blockIdx.x, b = blockIdx.z / parts, part = blockIdx.z - b * parts;
  const int G = nh / nkv;
  const int chunks = (G + 7) / 8;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y - kvh * chunks;
  const int h0 = kvh * G + chunk * 8;                           // first query head of this CTA
  const int nrows = min(8, G - chunk * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const bool consumer = warp < 4;
  pdl_trigger();
  if (smem_u32(smem_raw) & 1023u) {                             // the same in every CTA
    if (threadIdx.x == 0 && err) atomicExch(err, 5);
    return;
  }
  if (threadIdx.x == 0) {
    for (int i = 0; i < nst; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 4);                                  // one arrival per consumer warp
    }
    mbar_init(patched, NTHREADS);                               // the consumer threads
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&kmap) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&vmap) : "memory");
  }
  const bool late_wait = rope.fused && rope.write_kv;           // see the kernel above
  if (!late_wait) pdl_wait();
  const int row = cu_seqlens_q ? cu_seqlens_q[b] : b;
  const int p = positions[row];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int lo_al = lo / KT * KT;                               // tiles start on tile boundaries
  const int nkeys = p - lo_al + 1;
  const int pieces = splits * parts;
  int per = (nkeys + pieces - 1) / pieces;
  per = (per + KT - 1) / KT * KT;
  const int begin = lo_al + (part * splits + split) * per;
  const int end = min(p + 1, begin + per);
  const int first = max(begin, lo);                             // first visible key of this split
  const int ntiles = first < end ? (end - begin + KT - 1) / KT : 0;
  const int* tbl = block_table + (size_t)b * table_stride;
  int lp_base = 0;
  if (ntiles > 0) {
    const int lp0 = begin / page_size, nlp = (end - 1) / page_size - lp0 + 1;
    if (nlp <= tbl_cap) {
      for (int i = threadIdx.x; i < nlp; i += TMA_THREADS) stbl[i] = tbl[lp0 + i];
      tbl = stbl;
      lp_base = lp0;
    }
  }
  __syncthreads();                                              // barriers and table are set up

  float o[HD / 16][4];           // O^T: channels 16 mt + g (and + 8) of heads 2t, 2t + 1
#pragma unroll
  for (int mt = 0; mt < HD / 16; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};      // of heads 2t and 2t + 1

  if (!consumer) {
    // ---------------------------------------------------------------- the loader warp
    // A tile is 2 (K, V) x HALVES x boxes TMA boxes of box_rows keys; a lane keeps its boxes over
    // the tiles (two a lane where there are more than 32).  Tiles past the ring wait until the
    // four consumer warps have let go of their stage.  It reads only what earlier steps wrote
    // to the cache, so it does not wait for the kernel in front.
    const int box_rows = min(page_size, KT), boxes = KT / box_rows;
    const int ops = 2 * HALVES * boxes;
    const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
    int key_off[2];                                             // first key of the box in its tile
    uint32_t dst_off[2];
    int x_coord[2];
    bool is_v[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int op = min(lane + 32 * u, ops - 1);
      const int v = op / (HALVES * boxes), rem = op - v * HALVES * boxes;
      const int h = rem / boxes, bx = rem - h * boxes;
      is_v[u] = v != 0;
      key_off[u] = bx * box_rows;
      dst_off[u] = (uint32_t)v * TILE_BYTES + (uint32_t)h * HALF_BYTES +
                   (uint32_t)bx * (uint32_t)box_rows * 128u;
      x_coord[u] = kvh * HD + h * 64;
    }
    int st = 0;
    uint32_t ph = 0;                                            // of the ring's current round
    for (int it = 0; it < ntiles; ++it) {
      const int key0 = begin + it * KT;
      // (the wait for the round before the first one returns at once on a fresh barrier)
      if (!mbar_wait(&empty[st], ph ^ 1u, err, 6)) break;
      if (lane == 0) mbar_expect_tx(&full[st], STAGE_BYTES);
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (lane + 32 * u < ops) {
          const int c = key0 + key_off[u];
          int src_row = oob_row;                                // past the tensor: zeros
          if (c < end && c + box_rows > first) {
            const int lp = page_shift >= 0 ? c >> page_shift : c / page_size;
            const int page = tbl[lp - lp_base];
            if (page >= 0) src_row = page * page_size + (c - lp * page_size);
          }
          tma_load_2d(ring + (size_t)st * STAGE_BYTES + dst_off[u], is_v[u] ? &vmap : &kmap,
                      &full[st], x_coord[u], src_row);
        }
      }
      if (++st == nst) st = 0, ph ^= 1u;
    }
  } else {
    // ---------------------------------------------------------------- the consumer warps
    if (late_wait) pdl_wait();   // q (and the new k and v) come from the kernel in front
    // q as the 8-column operand: thread (g, t) holds channels 16 kc + 2t, +1 and + 8, + 9 of head g
    uint32_t qf[KCH][2];
    const bf16* qrow = q + (size_t)row * q_row_stride + (size_t)h0 * HD;
    bool patch = false;          // the last tile of this CTA gets the new token's k and v from here
    if (rope.fused && ntiles > 0) {
      const bf16* base = q + (size_t)row * q_row_stride;
      const int half = rope.rot >> 1, tail = HD - rope.rot;
      const float* cs = rope.table ? rope.table + (size_t)p * rope.rot : nullptr;
      for (int i = threadIdx.x; i < nrows * half; i += NTHREADS) {
        const int r = i / half, j = i - r * half;
        const float a = __bfloat162float(qrow[r * HD + j]);
        const float bb = __bfloat162float(qrow[r * HD + j + half]);
        const float c = cs[j], sn = cs[half + j];
        qs[r * HD + j] = __float2bfloat16_rn(a * c - bb * sn);
        qs[r * HD + j + half] = __float2bfloat16_rn(a * sn + bb * c);
      }
      for (int i = threadIdx.x; i < nrows * tail; i += NTHREADS) {
        const int r = i / tail, j = rope.rot + (i - r * tail);
        qs[r * HD + j] = qrow[r * HD + j];
      }
      if (rope.write_kv && p >= begin && p < end) {
        // this split holds the new token: its k (rotated) and v go into the tile of keys through
        // shared memory; the CTA of the first head chunk also writes them to the cache slot
        patch = true;
        const int lp = p / page_size;
        const size_t slot = (size_t)block_table[(size_t)b * table_stride + lp] * page_size +
                            (size_t)(p - lp * page_size);
        bf16* kd = kpages + slot * ((size_t)nkv * HD) + (size_t)kvh * HD;
        bf16* vd = vpages + slot * ((size_t)nkv * HD) + (size_t)kvh * HD;
        const bf16* kn = base + (size_t)(nh + kvh) * HD;
        const bf16* vn = base + (size_t)(nh + nkv + kvh) * HD;
        const bool store = chunk == 0;
        for (int j = threadIdx.x; j < half; j += NTHREADS) {
          const float a = __bfloat162float(kn[j]), bb = __bfloat162float(kn[j + half]);
          const float c = cs[j], sn = cs[half + j];
          const bf16 lo_v = __float2bfloat16_rn(a * c - bb * sn);
          const bf16 hi_v = __float2bfloat16_rn(a * sn + bb * c);
          knew[j] = lo_v, knew[j + half] = hi_v;
          if (store) kd[j] = lo_v, kd[j + half] = hi_v;
        }
        for (int j = rope.rot + threadIdx.x; j < HD; j += NTHREADS) {
          knew[j] = kn[j];
          if (store) kd[j] = kn[j];
        }
        for (int j = threadIdx.x; j < HD; j += NTHREADS) {
          vnew[j] = vn[j];
          if (store) vd[j] = vn[j];
        }
      }
      consumer_sync();           // q, and the new k and v, are in shared memory
      qrow = qs;
    }
#pragma unroll
    for (int kc = 0; kc < KCH; ++kc) {
      const uint32_t* r0 = reinterpret_cast<const uint32_t*>(
          qrow + (size_t)min(g, nrows - 1) * HD + kc * 16 + 2 * t);
      qf[kc][0] = g < nrows ? r0[0] : 0u;
      qf[kc][1] = g < nrows ? r0[4] : 0u;
    }
    const int mi = lane >> 3;
    int st = 0;
    uint32_t ph = 0;
    for (int it = 0; it < ntiles; ++it) {
      if (!mbar_wait(&full[st], ph, err, 4)) break;
      unsigned char* kt = ring + (size_t)st * STAGE_BYTES;
      unsigned char* vt = kt + TILE_BYTES;
      if (patch && it == ntiles - 1) {
        const int rp = p - (begin + it * KT);
        for (int j = threadIdx.x; j < HD; j += NTHREADS) {
          const uint32_t off = swz(rp, j & ~7) + (uint32_t)(j & 7) * 2u;
          *reinterpret_cast<bf16*>(kt + off) = knew[j];
          *reinterpret_cast<bf16*>(vt + off) = vnew[j];
        }
        // (a wait with a limit, like the one above: a warp that gave up there is not waited for)
        mbar_arrive(patched);
        if (!mbar_wait(patched, 0u, err, 4)) break;
      }
      const int col0 = begin + it * KT + warp * 16;
      if (col0 < end && col0 + 16 > first) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};   // S^T: keys col0 + g (and + 8) of heads 2t, 2t + 1
        {
          const int key = warp * 16 + (lane & 15), chsel = (lane >> 4) * 8;
#pragma unroll
          for (int kc = 0; kc < KCH; ++kc) {
            uint32_t a[4];
            ldsm_x4(a, kt + swz(key, kc * 16 + chsel));
            mma16816(s, a, qf[kc][0], qf[kc][1]);
          }
        }
        const int ka = col0 + g, kb = ka + 8;
        const bool va = ka >= first && ka < end, vb = kb >= first && kb < end;
        s[0] = va ? s[0] * scale_log2 : -INFINITY;
        s[1] = va ? s[1] * scale_log2 : -INFINITY;
        s[2] = vb ? s[2] * scale_log2 : -INFINITY;
        s[3] = vb ? s[3] * scale_log2 : -INFINITY;
        float mx[2] = {fmaxf(s[0], s[2]), fmaxf(s[1], s[3])};
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 4));
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 8));
          mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 16));
        }
        float corr[2], msub[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const float mnew = fmaxf(m[i], mx[i]);
          msub[i] = mnew == -INFINITY ? 0.f : mnew;
          corr[i] = fast_exp2(m[i] - msub[i]);
          m[i] = mnew;
        }
        const float p0 = fast_exp2(s[0] - msub[0]), p1 = fast_exp2(s[1] - msub[1]);
        const float p2 = fast_exp2(s[2] - msub[0]), p3 = fast_exp2(s[3] - msub[1]);
        l[0] = l[0] * corr[0] + (p0 + p2);
        l[1] = l[1] * corr[1] + (p1 + p3);
        if (__any_sync(0xffffffffu, corr[0] != 1.f || corr[1] != 1.f)) {
#pragma unroll
          for (int mt = 0; mt < HD / 16; ++mt) {
            o[mt][0] *= corr[0];
            o[mt][1] *= corr[1];
            o[mt][2] *= corr[0];
            o[mt][3] *= corr[1];
          }
        }
        // P^T as the 8-column operand: (keys 2t, 2t + 1 | + 8, + 9) of head g
        const uint32_t b0 = movmatrix_t(pack_bf16(p0, p1));
        const uint32_t b1 = movmatrix_t(pack_bf16(p2, p3));
        const int key = warp * 16 + (mi >> 1) * 8 + (lane & 7), chsel = (mi & 1) * 8;
#pragma unroll
        for (int mt = 0; mt < HD / 16; ++mt) {
          uint32_t a[4];
          ldsm_x4_t(a, vt + swz(key, mt * 16 + chsel));
          mma16816(o[mt], a, b0, b1);
        }
      }
      // this warp lets go of the stage
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[st]);
      if (++st == nst) st = 0, ph ^= 1u;
    }
  }
  __syncthreads();               // the ring is free: the merge buffers lie over it

  // a thread's sums cover its keys only: add up over the lanes that share its heads
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 4);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 8);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 16);
  }
  constexpr int SOP = HD + 4;    // head rows 4 banks apart: the scalar stores below do not collide
  float* so = reinterpret_cast<float*>(smem_raw);               // [4][8][SOP]
  float* sm = so + 4 * 8 * SOP;                                 // [4][8]
  float* sl = sm + 4 * 8;                                       // [4][8]
  float* cpart = sl + 4 * 8;                                    // [8][HD]: the CTA's partial
  float* cpart_m = cpart + 8 * HD;                              // [16]
  float* cpart_l = cpart_m + 16;                                // [16]
  float* cw = cpart_l + 16;                                     // [16][16], first [4][8] here
  float* cinv = cw + 256;                                       // [16]
  if (consumer) {
#pragma unroll
    for (int mt = 0; mt < HD / 16; ++mt) {
      float* base = so + (warp * 8 + 2 * t) * SOP + mt * 16 + g;
      base[0] = o[mt][0];
      base[SOP] = o[mt][1];
      base[8] = o[mt][2];
      base[SOP + 8] = o[mt][3];
    }
    if (g == 0) {
      sm[warp * 8 + 2 * t] = m[0];
      sm[warp * 8 + 2 * t + 1] = m[1];
      sl[warp * 8 + 2 * t] = l[0];
      sl[warp * 8 + 2 * t + 1] = l[1];
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int r = threadIdx.x & 7;
    const float mm = fmaxf(fmaxf(sm[r], sm[8 + r]), fmaxf(sm[16 + r], sm[24 + r]));
    cw[threadIdx.x] = mm == -INFINITY ? 0.f : exp2f(sm[threadIdx.x] - mm);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nrows * HD && consumer; i += NTHREADS) {
    const int r = i / HD, d = i - r * HD;
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) acc += cw[w * 8 + r] * so[(w * 8 + r) * SOP + d];
    float mm = -INFINITY, lsum = 0.f;
    if (d == 0 || splits == 1) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        mm = fmaxf(mm, sm[w * 8 + r]);
        lsum += cw[w * 8 + r] * sl[w * 8 + r];
      }
    }
    if (splits == 1 && parts > 1) {
      const size_t at = ((size_t)b * nh + h0 + r) * parts + part;
      po[at * HD + d] = acc;
      if (d == 0) {
        pml[at * 2] = mm;
        pml[at * 2 + 1] = lsum;
      }
    } else if (splits == 1) {
      out[((size_t)row * nh + h0 + r) * HD + d] =
          __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    } else {
      cpart[i] = acc;
      if (d == 0) {
        cpart_m[r] = mm;
        cpart_l[r] = lsum;
      }
    }
  }
  if (splits > 1) {
    float* part_o = parts > 1 ? po + (((size_t)b * nh + h0) * parts + part) * HD : nullptr;
    float* part_ml = parts > 1 ? pml + (((size_t)b * nh + h0) * parts + part) * 2 : nullptr;
    cluster_sync_all();          // also orders the weights above before they are overwritten
    if (splits <= 8)
      cluster_merge<8>(cpart, cpart_m, cpart_l, cw, cinv, out, nrows, splits, split, row, nh, h0,
                       consumer, part_o, part_ml, parts);
    else
      cluster_merge<16>(cpart, cpart_m, cpart_l, cw, cinv, out, nrows, splits, split, row, nh, h0,
                        consumer, part_o, part_ml, parts);
    cluster_sync_all();          // nobody leaves while a peer reads it
  }
}
#endif  // GF_HEAD_DIM % 64 == 0

// grid (nh, B), HD threads... one thread per output channel (HD <= 256).
__global__ void attn_decode_merge_kernel(const float* __restrict__ po,
                                         const float* __restrict__ pml,
                                         const int* __restrict__ cu_seqlens_q,
                                         bf16* __restrict__ out, int nh, int splits) {
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  pdl_trigger();
  pdl_wait();
  const size_t base = ((size_t)b * nh + head) * splits;
  // (eight parts' loads under way at a time: one after the other they were most of this kernel)
  float mm = -INFINITY;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, pml[(base + s) * 2]);
  float acc = 0.f, lsum = 0.f;
#pragma unroll 8
  for (int s = 0; s < splits; ++s) {
    const float ms = pml[(base + s) * 2];
    const float wgt = ms == -INFINITY ? 0.f : exp2f(ms - mm);
    acc += wgt * po[(base + s) * HD + d];
    lsum += wgt * pml[(base + s) * 2 + 1];
  }
  const int row = cu_seqlens_q ? cu_seqlens_q[b] : b;
  out[((size_t)row * nh + head) * HD + d] = __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
}

// ================================================================================== prefill
// grid (q tiles, nh, B): QT query rows of one head of one request.  Warp w owns rows
// 16 * MT * w .. + 16 * MT - 1: with MT = 2 every K/V fragment read from shared memory feeds two
// row tiles (four MMAs), which is what keeps the tensor pipe busier than the shared-memory pipe.
// Head sizes above 128 keep one row tile per warp (the output accumulator would not fit twice).
constexpr int PRE_STAGES = 2;
#ifndef GF_ATTN_MT
#define GF_ATTN_MT 1
#endif
constexpr int MT = HD <= 128 ? GF_ATTN_MT : 1;
constexpr int WROWS = 16 * MT;                 // query rows per warp
constexpr int QT = 4 * WROWS;                  // query rows per CTA

__global__ void __launch_bounds__(NTHREADS)
attn_prefill_kernel(const bf16* __restrict__ q, int q_row_stride, const bf16* __restrict__ kpages,
                    const bf16* __restrict__ vpages, const int* __restrict__ block_table,
                    int table_stride, const int* __restrict__ cu_seqlens_q,
                    const int* __restrict__ kv_lens, bf16* __restrict__ out, int nh, int nkv,
                    int page_size, int window, float scale_log2, int tbl_off, int tbl_cap) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);                 // [QT][ROW]
  bf16* ks = qs + QT * ROW;                                     // [STAGES][KT][ROW]
  bf16* vs = ks + PRE_STAGES * KT * ROW;
  const int b = blockIdx.z, head = blockIdx.y;
  pdl_trigger();
  pdl_wait();
  const int q_begin = cu_seqlens_q[b], q_len = cu_seqlens_q[b + 1] - q_begin;
  // later row tiles see more keys: they are handed out first so that the long ones do not trail
  const int r0 = (int)(gridDim.x - 1 - blockIdx.x) * QT;
  if (r0 >= q_len) return;
  const int kv_len = kv_lens[b];
  const int pos0 = kv_len - q_len;                              // position of the request's row 0
  const int kvh = head / (nh / nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
  const int* tbl = block_table + (size_t)b * table_stride;
  const size_t tok_stride = (size_t)nkv * HD;
  const int page_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
  const int rows = min(QT, q_len - r0);

  // the tile's queries -> shared memory (rows past the request's end are zero)
  {
    constexpr int CH = HD / 8;
    for (int i = threadIdx.x; i < QT * CH; i += NTHREADS) {
      const int r = i / CH, ch = i - r * CH;
      const bool ok = r < rows;
      const bf16* src = ok ? q + (size_t)(q_begin + r0 + r) * q_row_stride + (size_t)head * HD +
                                 ch * 8
                           : q;
      cp_async16(qs + r * ROW + ch * 8, src, ok);
    }
  }
  // keys this tile can see: from the window's start of its first row to its last row's position
  const int p_first = pos0 + r0, p_last = pos0 + r0 + rows - 1;
  const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
  const int begin = key_lo / KT * KT, end = p_last + 1;
  const int ntiles = (end - begin + KT - 1) / KT;
  int lp_base = 0;
  {
    const int lp0 = key_lo / page_size, nlp = (end - 1) / page_size - lp0 + 1;
    if (nlp <= tbl_cap) {
      int* stbl = reinterpret_cast<int*>(smem_raw + tbl_off);
      for (int i = threadIdx.x; i < nlp; i += NTHREADS) stbl[i] = tbl[lp0 + i];
      __syncthreads();
      tbl = stbl;
      lp_base = lp0;
    }
  }
  load_kv_tiles(ks, vs, kpages, vpages, tbl, lp_base, begin, key_lo, end, page_size, page_shift, tok_stride, kvh, threadIdx.x);
  cp_async_commit();

  float o[MT][HD / 8][4];
  float m[MT][2], l[MT][2];
  int lo2[MT][2], hi2[MT][2];                  // visibility bounds of this thread's rows
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) o[mt][n][0] = o[mt][n][1] = o[mt][n][2] = o[mt][n][3] = 0.f;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      m[mt][i] = -INFINITY;
      l[mt][i] = 0.f;
      const int r = warp * WROWS + mt * 16 + g + 8 * i;
      const int p = pos0 + r0 + r;
      hi2[mt][i] = r < rows ? p : -1;          // rows past the end see nothing
      lo2[mt][i] = window > 0 ? max(0, p - window + 1) : 0;
    }
  }
  const int warp_hi = min(p_last, pos0 + r0 + warp * WROWS + WROWS - 1);
  const int warp_lo = window > 0 ? max(0, pos0 + r0 + warp * WROWS - window + 1) : 0;
  const int mi = lane >> 3, lr = lane & 7;
  const bf16* qw = qs + (warp * WROWS + (mi & 1) * 8 + lr) * ROW + (mi >> 1) * 8;

  for (int it = 0; it < ntiles; ++it) {
    cp_async_wait<0>();
    __syncthreads();
    if (it + 1 < ntiles) {
      const int st = (it + 1) % PRE_STAGES;
      load_kv_tiles(ks + st * KT * ROW, vs + st * KT * ROW, kpages, vpages, tbl, lp_base,
                    begin + (it + 1) * KT, key_lo, end, page_size, page_shift, tok_stride, kvh, threadIdx.x);
    }
    cp_async_commit();
    const int st = it % PRE_STAGES;
    const int col0 = begin + it * KT;
    if (!(col0 <= warp_hi && col0 + KT > warp_lo && warp * WROWS < rows)) continue;
    const bf16* kt = ks + st * KT * ROW;
    const bf16* vt = vs + st * KT * ROW;
    float s[MT][8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int j = 0; j < 8; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f;
    // S = Q K^T: one K fragment (two key tiles) feeds every row tile of the warp
#pragma unroll
    for (int kc = 0; kc < KCH; ++kc) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) ldsm_x4(a[mt], qw + mt * 16 * ROW + kc * 16);
#pragma unroll
      for (int n2 = 0; n2 < 4; ++n2) {
        uint32_t kb[4];
        ldsm_x4(kb, kt + (n2 * 16 + (mi >> 1) * 8 + lr) * ROW + kc * 16 + (mi & 1) * 8);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma16816(s[mt][2 * n2], a[mt], kb[0], kb[1]);
          mma16816(s[mt][2 * n2 + 1], a[mt], kb[2], kb[3]);
        }
      }
    }
    // interior tile: every row of the warp sees all of its keys
    const int first_p = pos0 + r0 + warp * WROWS;
    const bool interior = col0 + KT - 1 <= first_p && warp * WROWS + WROWS <= rows &&
                          (window <= 0 || col0 >= first_p + WROWS - 1 - window + 1);
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      if (interior)
        softmax_update<8, false>(s[mt], o[mt], m[mt], l[mt], col0, lo2[mt], hi2[mt], scale_log2,
                                 lane);
      else
        softmax_update<8, true>(s[mt], o[mt], m[mt], l[mt], col0, lo2[mt], hi2[mt], scale_log2,
                                lane);
    }
    // O += P V
#pragma unroll
    for (int kc = 0; kc < 4; ++kc) {
      uint32_t a[MT][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        a[mt][0] = pack_bf16(s[mt][2 * kc][0], s[mt][2 * kc][1]);
        a[mt][1] = pack_bf16(s[mt][2 * kc][2], s[mt][2 * kc][3]);
        a[mt][2] = pack_bf16(s[mt][2 * kc + 1][0], s[mt][2 * kc + 1][1]);
        a[mt][3] = pack_bf16(s[mt][2 * kc + 1][2], s[mt][2 * kc + 1][3]);
      }
#pragma unroll
      for (int n2 = 0; n2 < HD / 16; ++n2) {
        uint32_t vb[4];
        ldsm_x4_t(vb, vt + (kc * 16 + (mi & 1) * 8 + lr) * ROW + n2 * 16 + (mi >> 1) * 8);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          mma16816(o[mt][2 * n2], a[mt], vb[0], vb[1]);
          mma16816(o[mt][2 * n2 + 1], a[mt], vb[2], vb[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  const int t = lane & 3;
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      float li = l[mt][i];
      li += __shfl_xor_sync(0xffffffffu, li, 1);
      li += __shfl_xor_sync(0xffffffffu, li, 2);
      const int r = warp * WROWS + mt * 16 + g + 8 * i;
      if (r >= rows) continue;
      const float inv = li > 0.f ? 1.f / li : 0.f;
      bf16* orow = out + ((size_t)(q_begin + r0 + r) * nh + head) * HD;
#pragma unroll
      for (int n = 0; n < HD / 8; ++n) {
        *reinterpret_cast<uint32_t*>(orow + n * 8 + 2 * t) =
            pack_bf16(o[mt][n][2 * i] * inv, o[mt][n][2 * i + 1] * inv);
      }
    }
  }
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_attn_head_dim() { return HD; }

// Bytes of scratch gf_attn_decode needs for B requests, nh heads and `splits` > 1 splits.
GF_EXPORT long long gf_attn_decode_scratch_bytes(int B, int nh, int splits) {
  return splits <= 1 ? 0 : (long long)B * nh * splits * (HD + 2) * (long long)sizeof(float);
}

// One query token per request (row cu_seqlens_q[b] of q / out; row b if cu_seqlens_q is null).
// splits > 1 with scratch (fp32, at least gf_attn_decode_scratch_bytes): partial results go through
// it; without scratch the splits (2, 4, 8 or 16) form a thread-block cluster and merge through
// distributed shared memory.
static int attn_decode_impl(const void* q, int q_row_stride, const void* kpages,
                            const void* vpages, const int* block_table, int table_stride,
                            const int* cu_seqlens_q, const int* positions, void* out,
                            void* scratch, int B, int nh, int nkv, int page_size, int window,
                            float scale, int splits, const RopeArgs& rope, void* stream) {
  if (B <= 0) return 0;
  if (nkv <= 0 || nh <= 0 || nh % nkv || splits < 1) return -3;
  auto st = (cudaStream_t)stream;
  const int G = nh / nkv, chunks = (G + 15) / 16;
  const size_t tiles = (size_t)2 * DEC_STAGES * KT * ROW * sizeof(bf16);
  const size_t merge = (size_t)(4 * 16 * (HD + 8) + 16 * HD + 2 * 4 * 16 + 32 + 256 + 16) * sizeof(float);
  const size_t work = ((tiles > merge ? tiles : merge) + 15) / 16 * 16;
  const int tbl_cap = table_stride < kMaxTableCopy ? table_stride : kMaxTableCopy;
  const size_t q_tile = (size_t)18 * HD * sizeof(bf16);        // fused mode: rotated q, new k and v
  const size_t smem = work + (size_t)tbl_cap * sizeof(int) + q_tile;
  // a kernel's attributes belong to a device: set them once on each device that is used
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevicesTracked) return -9;
  static std::mutex attr_lock;
  static bool attr_done[kMaxDevicesTracked] = {}, np_done[kMaxDevicesTracked] = {};
  {
    std::lock_guard<std::mutex> hold(attr_lock);
    if (!attr_done[dev]) {
      cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)(work + kMaxTableCopy * sizeof(int) + q_tile));
      if (e != cudaSuccess) return (int)e;
      attr_done[dev] = true;
    }
  }
  float* po = (float*)scratch;
  float* pml = po ? po + (size_t)B * nh * splits * HD : nullptr;
  dim3 grid(splits, nkv * chunks, B);
  if (splits > 1 && !scratch) {
    // cluster mode: the splits of a group merge through distributed shared memory
    if (splits != 2 && splits != 4 && splits != 8 && splits != 16) return -4;
    {
      std::lock_guard<std::mutex> hold(attr_lock);
      if (!np_done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel,
                                             cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return (int)e;
        np_done[dev] = true;
      }
    }
    return launch_kernel_cluster_dims(attn_decode_kernel, grid, dim3(NTHREADS), smem, st, splits,
                                      true, (const bf16*)q, q_row_stride, (const bf16*)kpages,
                                      (const bf16*)vpages, block_table, table_stride,
                                      cu_seqlens_q, positions, (bf16*)out, (float*)nullptr,
                                      (float*)nullptr, nh, nkv, page_size, window, scale * LOG2E,
                                      splits, 2, (int)work, tbl_cap, rope);
  }
  const int fused = (size_t)B * nkv * chunks <= (size_t)kMaxDecodeGroups ? 1 : 0;
  int rc = launch_kernel(attn_decode_kernel, grid, dim3(NTHREADS), smem, st, (const bf16*)q,
                         q_row_stride, (const bf16*)kpages, (const bf16*)vpages, block_table,
                         table_stride, cu_seqlens_q, positions, (bf16*)out, po, pml, nh, nkv,
                         page_size, window, scale * LOG2E, splits, fused, (int)work, tbl_cap, rope);
  if (rc || splits == 1 || fused) return rc;
  return launch_kernel(attn_decode_merge_kernel, dim3(nh, B), dim3(HD), 0, st, (const float*)po,
                       (const float*)pml, cu_seqlens_q, (bf16*)out, nh, splits);
}

// The TMA kernel where it serves the case: head sizes that are a multiple of 64, page sizes that
// are a multiple of 8 and divide (or are a multiple of) the 64-key tile, 1 split or a cluster of
// 2, 4, 8 or 16.  -6: not served (the caller takes gf_attn_decode / gf_attn_decode_rope).
// `stages`: depth of the ring of tiles (2 .. 6, cut to what shared memory holds; 3 lets two CTAs
// share an SM).  `err` receives 4 or 6 if a wait for a tile or for a free stage ran out.
GF_EXPORT int gf_attn_decode_tma(const void* q, int q_row_stride, void* kpages, void* vpages,
                                 int num_pages, const int* block_table, int table_stride,
                                 const int* cu_seqlens_q, const int* positions, void* out, int B,
                                 int nh, int nkv, int page_size, int window, float scale,
                                 int splits, int stages, const float* rope_table, int rot,
                                 int fused, int write_kv, int* err, void* stream, int parts,
                                 void* scratch) {
#if GF_HEAD_DIM % 64 == 0
  if (B <= 0) return 0;
  if (nh % nkv || splits < 1 || parts < 1 || (parts > 1 && !scratch)) return -3;
  if ((long long)B * parts > 65535) return -6;
  if (fused && (rot < 0 || rot > HD || rot % 2 || (!rope_table && rot))) return -3;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8 && splits != 16) return -6;
  if (page_size % 8 || (KT % page_size && page_size % KT) || num_pages <= 0) return -6;
  if (((uintptr_t)q & 3) || q_row_stride % 2 || ((uintptr_t)kpages & 15) ||
      ((uintptr_t)vpages & 15))
    return -6;
  const long long slots = (long long)num_pages * page_size;
  if (slots >= (1ll << 31) - KT) return -6;
  const int box_rows = page_size < KT ? page_size : KT;
  CUtensorMap mk, mv;
  if (!make_map(&mk, kpages, (int)slots, nkv * HD, nkv * HD, box_rows)) return -6;
  if (!make_map(&mv, vpages, (int)slots, nkv * HD, nkv * HD, box_rows)) return -6;
  auto st = (cudaStream_t)stream;
  const int G = nh / nkv, chunks = (G + 7) / 8;
  const int tbl_cap = table_stride < kMaxTableCopyTma ? table_stride : kMaxTableCopyTma;
  const size_t small = (2 * TMAX_STAGES + 1) * sizeof(uint64_t) + (size_t)10 * HD * sizeof(bf16);
  const size_t room = (size_t)227 * 1024 - small - kMaxTableCopyTma * sizeof(int);
  const int most = (int)(room / STAGE_BYTES) < TMAX_STAGES ? (int)(room / STAGE_BYTES) : TMAX_STAGES;
  const int nst = stages < 2 ? 2 : stages > most ? most : stages;
  const size_t smem = (size_t)nst * STAGE_BYTES + small + (size_t)tbl_cap * sizeof(int);
  static OncePerDevice attrs;
  if (int rc = attrs.run([&] {
        cudaError_t e = cudaFuncSetAttribute(
            attn_decode_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
            (int)((size_t)most * STAGE_BYTES + small + kMaxTableCopyTma * sizeof(int)));
        if (e == cudaSuccess)
          e = cudaFuncSetAttribute(attn_decode_tma_kernel,
                                   cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        return e;
      }))
    return rc;
  const RopeArgs rope{fused ? rope_table : nullptr, fused ? rot : 0, fused ? 1 : 0,
                      fused && write_kv ? 1 : 0};
  // `parts` > 1 (few requests with many keys): that many clusters share a request's keys; they
  // leave their results in `scratch` (gf_attn_decode_scratch_bytes(B, nh, parts) bytes) and a
  // second kernel adds them up
  float* po = (float*)scratch;
  float* pml = po ? po + (size_t)B * nh * parts * HD : nullptr;
  dim3 grid(splits, nkv * chunks, B * parts);
  int rc = launch_kernel_cluster_dims(attn_decode_tma_kernel, grid, dim3(TMA_THREADS), smem, st,
                                      splits, true, mk, mv, (const bf16*)q, q_row_stride,
                                      (bf16*)kpages, (bf16*)vpages, block_table, table_stride,
                                      cu_seqlens_q, positions, (bf16*)out, nh, nkv, page_size,
                                      window, scale * LOG2E, splits, (int)slots, tbl_cap, nst, err,
                                      rope, parts, po, pml);
  if (rc || parts == 1) return rc;
  return launch_kernel(attn_decode_merge_kernel, dim3(nh, B), dim3(HD), 0, st, (const float*)po,
                       (const float*)pml, cu_seqlens_q, (bf16*)out, nh, parts);
#else
  return -6;
#endif
}

GF_EXPORT int gf_attn_decode(const void* q, int q_row_stride, const void* kpages,
                             const void* vpages, const int* block_table, int table_stride,
                             const int* cu_seqlens_q, const int* positions, void* out,
                             void* scratch, int B, int nh, int nkv, int page_size, int window,
                             float scale, int splits, void* stream) {
  return attn_decode_impl(q, q_row_stride, kpages, vpages, block_table, table_stride,
                          cu_seqlens_q, positions, out, scratch, B, nh, nkv, page_size, window,
                          scale, splits, RopeArgs{nullptr, 0, 0, 0}, stream);
}

// The same with the rotation of q and k and the write of the new k and v to the cache done by the
// attention kernel itself: `q` points at rows [q | k | v] as the q/k/v product left them;
// `rope_table` row p holds cos | sin of position p over `rot` channels (null: no rotation).
GF_EXPORT int gf_attn_decode_rope(const void* q, int q_row_stride, void* kpages, void* vpages,
                                  const int* block_table, int table_stride,
                                  const int* cu_seqlens_q, const int* positions, void* out,
                                  void* scratch, int B, int nh, int nkv, int page_size,
                                  int window, float scale, int splits, const float* rope_table,
                                  int rot, int write_kv, void* stream) {
  if (rot < 0 || rot > HD || rot % 2 || (!rope_table && rot)) return -3;
  return attn_decode_impl(q, q_row_stride, kpages, vpages, block_table, table_stride,
                          cu_seqlens_q, positions, out, scratch, B, nh, nkv, page_size, window,
                          scale, splits, RopeArgs{rope_table, rot, 1, write_kv ? 1 : 0}, stream);
}

GF_EXPORT int gf_attn_prefill(const void* q, int q_row_stride, const void* kpages,
                              const void* vpages, const int* block_table, int table_stride,
                              const int* cu_seqlens_q, const int* kv_lens, void* out, int B,
                              int max_q_len, int nh, int nkv, int page_size, int window,
                              float scale, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (nh % nkv) return -3;
  auto st = (cudaStream_t)stream;
  const size_t work = (size_t)(QT + 2 * PRE_STAGES * KT) * ROW * sizeof(bf16);
  const int tbl_cap = table_stride < kMaxTableCopy ? table_stride : kMaxTableCopy;
  const size_t smem = work + (size_t)tbl_cap * sizeof(int);
  static OncePerDevice attrs;
  if (int rc = attrs.run([&] {
        return cudaFuncSetAttribute(attn_prefill_kernel,
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)(work + kMaxTableCopy * sizeof(int)));
      }))
    return rc;
  dim3 grid((max_q_len + QT - 1) / QT, nh, B);
  return launch_kernel(attn_prefill_kernel, grid, dim3(NTHREADS), smem, st, (const bf16*)q,
                       q_row_stride, (const bf16*)kpages, (const bf16*)vpages, block_table,
                       table_stride, cu_seqlens_q, kv_lens, (bf16*)out, nh, nkv, page_size, window,
                       scale * LOG2E, (int)work, tbl_cap);
}

// ----------------------------------------------------------------------------- no allocation
// gf_attn_decode with scratch of its own; see attention_no_alloc.h for who needs it and the rules.
#include <stdio.h>

#include "attention_no_alloc.h"

namespace {

// The scratch of gf_attn_decode_static.  In host code this name is only a handle for
// cudaGetSymbolAddress, never an address a kernel could use.
static __device__ __align__(256) unsigned char g_static_scratch[GF_ATTN_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = kMaxDevicesTracked;
void* g_static_scratch_addr[kMaxDevices] = {};     // device address per device, found on first use
std::mutex g_static_lock;                          // guards the look-up: first calls may coincide
thread_local char g_static_error[256] = "";

}  // namespace

GF_EXPORT const char* gf_attn_decode_static_error(void) { return g_static_error; }

GF_EXPORT int gf_attn_decode_static(const void* q, int q_row_stride, const void* kpages,
                                    const void* vpages, const int* block_table, int table_stride,
                                    const int* cu_seqlens_q, const int* positions, void* out,
                                    int B, int nh, int nkv, int page_size, int window, float scale,
                                    int splits, void* stream) {
  g_static_error[0] = 0;
  const long long need = gf_attn_decode_scratch_bytes(B, nh, splits);
  if (need > (long long)GF_ATTN_STATIC_SCRATCH_BYTES) {
    snprintf(g_static_error, sizeof g_static_error,
             "gf_attn_decode_static: %d requests x %d heads x %d splits x head size %d need %lld "
             "bytes of scratch; the built-in array holds %u",
             B, nh, splits, HD, need, (unsigned)GF_ATTN_STATIC_SCRATCH_BYTES);
    return GF_ATTN_STATIC_TOO_LARGE;
  }
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    snprintf(g_static_error, sizeof g_static_error,
             "gf_attn_decode_static: no usable current device (cudaGetDevice: %s, device %d)",
             cudaGetErrorString(e), dev);
    return e != cudaSuccess ? (int)e : -9;
  }
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> hold(g_static_lock);
    if (!g_static_scratch_addr[dev]) {
      // once per device, with that device current: the array's address on this device
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p) {
        snprintf(g_static_error, sizeof g_static_error,
                 "gf_attn_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                 cudaGetErrorString(e));
        return e != cudaSuccess ? (int)e : -9;
      }
      g_static_scratch_addr[dev] = p;
    }
    scratch = g_static_scratch_addr[dev];
  }
  return gf_attn_decode(q, q_row_stride, kpages, vpages, block_table, table_stride, cu_seqlens_q,
                        positions, out, splits > 1 ? scratch : nullptr, B, nh, nkv, page_size,
                        window, scale, splits, stream);
}
