// Paged grouped-query attention with plain fp32 arithmetic: the kernel of the 32-bit path, and the
// fall-back of the bf16 path for head sizes the tensor-core kernels do not take.
//
// One warp owns one (token, query head).  The token's absolute position p decides what it sees:
// keys lo..p with lo = max(0, p - window + 1) when window > 0, else 0.  Keys are visited in order in
// groups of 32 starting at lo, so a row's result depends only on (lo, p) and the cache contents,
// never on how the step was cut or what else is in the batch.  Running maximum, sum and the output
// accumulator are fp32.
#include "common.cuh"

namespace gf {

constexpr int kMaxHeadDim = 256;
constexpr int kWarps = 4;

template <typename T>
__global__ void paged_attention_simt_kernel(
    const T* __restrict__ q, int q_row_stride, const T* __restrict__ kpages,
    const T* __restrict__ vpages, const int* __restrict__ block_table, int table_stride,
    const int* __restrict__ seq_of_token, const int* __restrict__ positions, T* __restrict__ out,
    int num_pairs, int nh, int nkv, int hd, int page_size, int window, float scale) {
  extern __shared__ float qs_all[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x * kWarps + warp;
  if (pair >= num_pairs) return;
  float* qs = qs_all + warp * hd;
  const int t = pair / nh, n = pair - t * nh;
  const int kvh = n / (nh / nkv);
  const int b = seq_of_token[t];
  const int p = positions[t];
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int* tbl = block_table + (size_t)b * table_stride;
  const T* qrow = q + (size_t)t * q_row_stride + (size_t)n * hd;
  for (int d = lane; d < hd; d += 32) qs[d] = to_f32(qrow[d]);
  __syncwarp();

  float acc[kMaxHeadDim / 32];
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const size_t tok_stride = (size_t)nkv * hd;

  for (int c0 = lo; c0 <= p; c0 += 32) {
    const int c = c0 + lane;
    const bool valid = c <= p;
    int slot = 0;
    float s = -INFINITY;
    if (valid) {
      const int page = tbl[c / page_size];
      slot = page * page_size + c % page_size;
      const T* krow = kpages + (size_t)slot * tok_stride + (size_t)kvh * hd;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot = fmaf(qs[d], to_f32(krow[d]), dot);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pexp = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);          // m = -inf on the first group: corr = 0
    l = l * corr + warp_sum(pexp);
#pragma unroll
    for (int i = 0; i < kMaxHeadDim / 32; ++i) acc[i] *= corr;
    const int nvalid = min(32, p - c0 + 1);
    for (int j = 0; j < nvalid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, pexp, j);
      const int sj = __shfl_sync(0xffffffffu, slot, j);
      const T* vrow = vpages + (size_t)sj * tok_stride + (size_t)kvh * hd;
#pragma unroll
      for (int i = 0; i < kMaxHeadDim / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vrow[d]), acc[i]);
      }
    }
    m = m_new;
  }
  T* orow = out + ((size_t)t * nh + n) * hd;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < kMaxHeadDim / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_f32<T>(acc[i] * inv);
  }
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

// q: rows of q_row_stride elements whose first nh*hd hold the query heads.  kpages/vpages:
// [num_pages, page_size, nkv, hd].  out: [T, nh, hd] packed.  Returns -3 for head sizes it refuses.
GF_EXPORT int gf_paged_attention_simt(const void* q, int q_row_stride, const void* kpages,
                                      const void* vpages, const int* block_table, int table_stride,
                                      const int* seq_of_token, const int* positions, void* out,
                                      int T, int nh, int nkv, int hd, int page_size, int window,
                                      float scale, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (hd > kMaxHeadDim || hd <= 0 || nh % nkv) return -3;
  const int pairs = T * nh;
  const int blocks = (pairs + kWarps - 1) / kWarps;
  const size_t smem = (size_t)kWarps * hd * sizeof(float);
  auto st = (cudaStream_t)stream;
  if (dtype == GF_F32)
    paged_attention_simt_kernel<float><<<blocks, kWarps * 32, smem, st>>>(
        (const float*)q, q_row_stride, (const float*)kpages, (const float*)vpages, block_table,
        table_stride, seq_of_token, positions, (float*)out, pairs, nh, nkv, hd, page_size, window,
        scale);
  else
    paged_attention_simt_kernel<__nv_bfloat16><<<blocks, kWarps * 32, smem, st>>>(
        (const __nv_bfloat16*)q, q_row_stride, (const __nv_bfloat16*)kpages,
        (const __nv_bfloat16*)vpages, block_table, table_stride, seq_of_token, positions,
        (__nv_bfloat16*)out, pairs, nh, nkv, hd, page_size, window, scale);
  return launch_status();
}
