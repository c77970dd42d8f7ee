// Next-token choice from fp32 logits: arg-max with the lowest index winning ties, and temperature
// sampling by inverse CDF in index order.  The reference has arg-max only
// (ginfer/core/op/kernels/cuda/argmax_kernel.cu:63-98), compares in fp32, and does not fix the
// winner of a tie; here the lowest index wins so that greedy decoding does not depend on the batch.
#include "common.cuh"

namespace gf {

constexpr int kThreads = 256;

__device__ __forceinline__ void better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}

// Row arg-max; every thread returns the winner.  NaN never wins.
__device__ int row_argmax(const float* __restrict__ x, int V, float* sval, int* sidx,
                          float* max_out) {
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = threadIdx.x; j < V; j += blockDim.x) better(v, idx, x[j], j);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    better(v, idx, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sval[warp] = v; sidx[warp] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) better(v, idx, sval[w], sidx[w]);
    if (idx == 0x7fffffff) idx = 0;
    sval[0] = v; sidx[0] = idx;
  }
  __syncthreads();
  *max_out = sval[0];
  const int r = sidx[0];
  __syncthreads();
  return r;
}

// Arg-max of long rows in two stages inside one launch: every block reduces one chunk of a row and
// parks its (value, index); the block that finishes a row last (counted with an atomic that it
// resets for the next launch) reduces the parked pairs.  kMaxRows bounds the counters.
constexpr int kChunk = 4096;
constexpr int kMaxRows = 4096;
__device__ unsigned int g_row_done[kMaxRows];

__global__ void argmax_kernel(const float* __restrict__ logits, int* __restrict__ out, int V,
                              float* __restrict__ pval, int* __restrict__ pidx) {
  __shared__ float sval[kThreads / 32];
  __shared__ int sidx[kThreads / 32];
  __shared__ bool last;
  const int row = blockIdx.y, chunk = blockIdx.x, nchunks = gridDim.x;
  pdl_trigger();
  pdl_wait();
  const float* x = logits + (size_t)row * V;
  const int j0 = chunk * kChunk, j1 = min(V, j0 + kChunk);
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = j0 + threadIdx.x; j < j1; j += blockDim.x) better(v, idx, x[j], j);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    better(v, idx, ov, oi);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sval[warp] = v; sidx[warp] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) better(v, idx, sval[w], sidx[w]);
    if (nchunks == 1) {
      out[row] = idx == 0x7fffffff ? 0 : idx;
      last = false;
    } else {
      pval[(size_t)row * nchunks + chunk] = v;
      pidx[(size_t)row * nchunks + chunk] = idx;
      __threadfence();
      const unsigned int done = atomicAdd(&g_row_done[row], 1u);
      last = done == (unsigned int)nchunks - 1;
    }
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  v = -INFINITY;
  idx = 0x7fffffff;
  for (int c = threadIdx.x; c < nchunks; c += blockDim.x)
    better(v, idx, __ldcg(pval + (size_t)row * nchunks + c), __ldcg(pidx + (size_t)row * nchunks + c));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    better(v, idx, ov, oi);
  }
  __syncthreads();
  if (lane == 0) { sval[warp] = v; sidx[warp] = idx; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (blockDim.x >> 5); ++w) better(v, idx, sval[w], sidx[w]);
    out[row] = idx == 0x7fffffff ? 0 : idx;
    g_row_done[row] = 0;                       // ready for the next launch
  }
}

// temperature[r] <= 0: arg-max.  Otherwise w_j = expf((x_j - max) / temperature); thread i owns the
// contiguous chunk i of the row; the chosen index is the first j with sum_{k<=j} w_k >= u * total,
// the sums taken chunk by chunk in index order.
__global__ void sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperature,
                              const float* __restrict__ u, int* __restrict__ out, int V) {
  __shared__ float sval[kThreads / 32];
  __shared__ int sidx[kThreads / 32];
  __shared__ float part[kThreads];
  __shared__ float s_target;
  __shared__ int s_owner;
  const float* x = logits + (size_t)blockIdx.x * V;
  float mx;
  const int amax = row_argmax(x, V, sval, sidx, &mx);
  const float temp = temperature[blockIdx.x];
  if (!(temp > 0.f)) {
    if (threadIdx.x == 0) out[blockIdx.x] = amax;
    return;
  }
  const float inv_t = 1.f / temp;
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int j0 = min(V, (int)threadIdx.x * chunk), j1 = min(V, j0 + chunk);
  float s = 0.f;
  for (int j = j0; j < j1; ++j) s += expf((x[j] - mx) * inv_t);
  part[threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float total = 0.f;
    for (int i = 0; i < blockDim.x; ++i) total += part[i];
    const float target = u[blockIdx.x] * total;
    float cum = 0.f;
    int owner = -1;
    for (int i = 0; i < blockDim.x; ++i) {
      if (cum + part[i] >= target && part[i] > 0.f) { owner = i; break; }
      cum += part[i];
    }
    s_owner = owner;
    s_target = target - cum;      // what is left to cover inside the owner's chunk
  }
  __syncthreads();
  if (s_owner < 0) {              // rounding pushed the target past the total: take the arg-max
    if (threadIdx.x == 0) out[blockIdx.x] = amax;
    return;
  }
  if ((int)threadIdx.x == s_owner) {
    float cum = 0.f;
    int pick = -1, last = j0;
    for (int j = j0; j < j1; ++j) {
      const float w = expf((x[j] - mx) * inv_t);
      if (w > 0.f) last = j;
      cum += w;
      if (cum >= s_target && w > 0.f) { pick = j; break; }
    }
    out[blockIdx.x] = pick >= 0 ? pick : last;
  }
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

// scratch: room for 2 * R * ceil(V / 4096) 32-bit words (parked pairs); may be null when V <= 4096.
// dst[dst_idx[i]] = src[src_idx[i]]: tokens chosen in the step before are fed to the next step
// on the device, before the host has seen them.
__global__ void scatter_tokens_kernel(int* __restrict__ dst, const int* __restrict__ dst_idx,
                                      const int* __restrict__ src, const int* __restrict__ src_idx,
                                      int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[dst_idx[i]] = src[src_idx[i]];
}

GF_EXPORT int gf_scatter_tokens(int* dst, const int* dst_idx, const int* src, const int* src_idx,
                                int n, void* stream) {
  if (n <= 0) return 0;
  scatter_tokens_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(dst, dst_idx, src,
                                                                            src_idx, n);
  return (int)cudaGetLastError();
}

GF_EXPORT int gf_argmax(const float* logits, int* out, int R, int V, void* scratch, void* stream) {
  if (R <= 0) return 0;
  if (R > kMaxRows) return -5;
  const int nchunks = (V + kChunk - 1) / kChunk;
  if (nchunks > 1 && !scratch) return -4;
  float* pval = (float*)scratch;
  int* pidx = (int*)scratch + (size_t)R * nchunks;
  return launch_kernel(argmax_kernel, dim3(nchunks, R), dim3(kThreads), 0, (cudaStream_t)stream,
                       logits, out, V, pval, pidx);
}

GF_EXPORT int gf_sample(const float* logits, const float* temperature, const float* u, int* out,
                        int R, int V, void* stream) {
  if (R <= 0) return 0;
  sample_kernel<<<R, kThreads, 0, (cudaStream_t)stream>>>(logits, temperature, u, out, V);
  return launch_status();
}
