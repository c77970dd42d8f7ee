// Memory-bound kernels of the step: embedding gather, fused residual-add + RMSNorm (optionally on
// selected rows), rotary encoding fused with the K/V page write, SiLU(gate) * up.
// Every kernel is a template over the activation type (float for the 32-bit path, bf16 for the
// serving path); arithmetic is fp32 in both.
#include "common.cuh"

namespace gf {

// ----------------------------------------------------------------------------- embedding
// out[t, :] = W[ids[t], :], copied in `unit`-byte words (16 when rows allow it).
template <typename V>
__global__ void embedding_kernel(const int* __restrict__ ids, const V* __restrict__ w,
                                 V* __restrict__ out, int words_per_row) {
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  const V* src = w + (size_t)ids[t] * words_per_row;
  V* dst = out + (size_t)t * words_per_row;
  for (int i = threadIdx.x; i < words_per_row; i += blockDim.x) dst[i] = src[i];
}

// ----------------------------------------------------------------------------- add + rmsnorm
// s = x[src] (+ delta[src]) formed and kept in fp32 (the residual stream is fp32 in both paths: x
// is the activation type only for the embedding's output); normed = s * gamma / rms with
// rms = sqrtf(sum(s^2) / H + eps), stored in the activation type.  `rows` (nullable) selects source
// rows.  One block per row; the row is parked in shared memory between the two passes.
template <typename XT, typename T, typename G>
__global__ void add_rmsnorm_kernel(const XT* __restrict__ x, const T* __restrict__ delta,
                                   const G* __restrict__ gamma, const int* __restrict__ rows,
                                   float* __restrict__ sum_out, T* __restrict__ normed, int H,
                                   float eps) {
  extern __shared__ float row[];                    // the row, then gamma: 2 * H floats
  __shared__ float scratch[33];
  float* gam = row + H;
  const int r = blockIdx.x;
  pdl_trigger();
  for (int j = threadIdx.x; j < H; j += blockDim.x) gam[j] = to_f32(gamma[j]);   // weights: no wait
  pdl_wait();
  const size_t src = (size_t)(rows ? rows[r] : r) * H;
  const size_t dst = (size_t)r * H;
  float ss = 0.f;
#pragma unroll 4
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float s = to_f32(x[src + j]);
    if (delta) s += to_f32(delta[src + j]);
    if (sum_out) sum_out[dst + j] = s;
    row[j] = s;
    ss += s * s;
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll 4
  for (int j = threadIdx.x; j < H; j += blockDim.x)
    normed[dst + j] = from_f32<T>(row[j] * gam[j] / rms);
}


// The same with 8 channels (an octet) per access and the row kept in registers: OPT octets a
// thread, one block per row.  Needs H to be a multiple of 8 and 16-byte aligned rows; the launcher
// checks.  Per row this moves what the definition needs and nothing else: x (and delta) in, the
// sum and the normalised row out.
template <typename T> struct Oct;                       // 8 values of T <-> 8 floats
template <> struct Oct<float> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
  }
};
template <> struct Oct<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x, v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
  }
};

template <typename XT, typename T, typename G, int OPT>
__global__ void add_rmsnorm_vec_kernel(const XT* __restrict__ x, const T* __restrict__ delta,
                                       const G* __restrict__ gamma, const int* __restrict__ rows,
                                       float* __restrict__ sum_out, T* __restrict__ normed, int H,
                                       float eps) {
  __shared__ float scratch[33];
  const int r = blockIdx.x, noct = H >> 3;
  pdl_trigger();
  float gam[OPT][8], s[OPT][8];
#pragma unroll
  for (int u = 0; u < OPT; ++u) {                       // weights: before the wait
    const int o = threadIdx.x + u * blockDim.x;
    if (o < noct) Oct<G>::load(gamma + o * 8, gam[u]);
  }
  pdl_wait();
  const size_t src = (size_t)(rows ? rows[r] : r) * H;
  const size_t dst = (size_t)r * H;
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int o = threadIdx.x + u * blockDim.x;
    if (o < noct) {
      Oct<XT>::load(x + src + o * 8, s[u]);
      if (delta) {
        float d[8];
        Oct<T>::load(delta + src + o * 8, d);
#pragma unroll
        for (int i = 0; i < 8; ++i) s[u][i] += d[i];
      }
      if (sum_out) Oct<float>::store(sum_out + dst + o * 8, s[u]);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += s[u][i] * s[u][i];
    }
  }
  ss = block_sum(ss, scratch);
  const float rms = sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int u = 0; u < OPT; ++u) {
    const int o = threadIdx.x + u * blockDim.x;
    if (o < noct) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = s[u][i] * gam[u][i] / rms;
      Oct<T>::store(normed + dst + o * 8, v);
    }
  }
}

// ----------------------------------------------------------------------------- rope + KV write
// qkv[t] = [q heads | k heads | v heads], each head hd wide.  The first `rot` channels of every q
// and k head are rotated in pairs (j, j + rot/2) by the angle of positions[t]; table row p holds
// cos[0..rot/2) then sin[0..rot/2).  q is rotated in place.  If slot_mapping is given, rotated k
// and plain v go to token slot slot_mapping[t] of the K and V pages (slot < 0: skipped).
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride,
                                     const float* __restrict__ table, int rot,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, T* __restrict__ kpages,
                                     T* __restrict__ vpages, int nh, int nkv, int hd) {
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  T* rowp = qkv + (size_t)t * row_stride;
  const int half = rot >> 1;
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  T* kdst = slot >= 0 ? kpages + (size_t)slot * nkv * hd : nullptr;
  T* vdst = slot >= 0 ? vpages + (size_t)slot * nkv * hd : nullptr;
  const float* cs = table ? table + (size_t)positions[t] * rot : nullptr;
  // The launch gives one thread per rotated pair and per copied channel when they number at most
  // 1024, so the loops below run once and a thread's loads are all issued before its stores.
  const int npairs = (nh + nkv) * half;
  for (int i = threadIdx.x; i < npairs; i += blockDim.x) {
    const int head = i / half, j = i - head * half;
    const float c = cs[j], s = cs[half + j];
    T* h = rowp + (size_t)head * hd;
    const float a = to_f32(h[j]), b = to_f32(h[j + half]);
    const T lo = from_f32<T>(a * c - b * s), hi = from_f32<T>(a * s + b * c);
    if (head < nh) {
      h[j] = lo;
      h[j + half] = hi;
    } else if (kdst) {
      T* kd = kdst + (size_t)(head - nh) * hd;
      kd[j] = lo;
      kd[j + half] = hi;
    }
  }
  if (!kdst) return;
  // channels of k beyond the rotated ones, and all of v
  const int tail = hd - rot;
  const int nk_tail = nkv * tail;
  for (int i = threadIdx.x; i < nk_tail; i += blockDim.x) {
    const int head = i / tail, j = rot + (i - head * tail);
    kdst[(size_t)head * hd + j] = rowp[(size_t)(nh + head) * hd + j];
  }
  const T* vsrc = rowp + (size_t)(nh + nkv) * hd;
  for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) vdst[i] = vsrc[i];
}

// The same with 16-byte accesses: a thread rotates VEC consecutive pairs (VEC = 8 bf16 or 4 fp32)
// or copies VEC channels.  Needs rot/2, hd and the row stride to be multiples of VEC and 16-byte
// aligned pointers; the launcher checks.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, int row_stride,
                                         const float* __restrict__ table, int rot,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ slot_mapping,
                                         T* __restrict__ kpages, T* __restrict__ vpages, int nh,
                                         int nkv, int hd) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const int t = blockIdx.x;
  pdl_trigger();
  pdl_wait();
  T* rowp = qkv + (size_t)t * row_stride;
  const int half = rot >> 1;
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  T* kdst = slot >= 0 ? kpages + (size_t)slot * nkv * hd : nullptr;
  T* vdst = slot >= 0 ? vpages + (size_t)slot * nkv * hd : nullptr;
  const float* cs = table ? table + (size_t)positions[t] * rot : nullptr;
  const int per_head = half / VEC;
  const int nrot = (nh + nkv) * per_head;                 // vector pairs to rotate
  const int tailv = (hd - rot) / VEC;                     // unrotated vectors per k head
  const int ncopy = kdst ? nkv * tailv + nkv * hd / VEC : 0;
  for (int i = threadIdx.x; i < nrot + ncopy; i += blockDim.x) {
    if (i < nrot) {
      const int head = i / per_head, j = (i - head * per_head) * VEC;
      T* h = rowp + (size_t)head * hd;
      const uint4 ra = *reinterpret_cast<const uint4*>(h + j);
      const uint4 rb = *reinterpret_cast<const uint4*>(h + j + half);
      const T* a = reinterpret_cast<const T*>(&ra);
      const T* b = reinterpret_cast<const T*>(&rb);
      T lo[VEC], hi[VEC];
#pragma unroll
      for (int k = 0; k < VEC; ++k) {
        const float c = cs[j + k], s = cs[half + j + k];
        const float x = to_f32(a[k]), y = to_f32(b[k]);
        lo[k] = from_f32<T>(x * c - y * s);
        hi[k] = from_f32<T>(x * s + y * c);
      }
      T* dst = head < nh ? h : (kdst ? kdst + (size_t)(head - nh) * hd : nullptr);
      if (dst) {
        *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(lo);
        *reinterpret_cast<uint4*>(dst + j + half) = *reinterpret_cast<const uint4*>(hi);
      }
    } else {
      const int c = i - nrot;
      if (c < nkv * tailv) {
        const int head = c / tailv, j = rot + (c - head * tailv) * VEC;
        *reinterpret_cast<uint4*>(kdst + (size_t)head * hd + j) =
            *reinterpret_cast<const uint4*>(rowp + (size_t)(nh + head) * hd + j);
      } else {
        const int j = (c - nkv * tailv) * VEC;
        *reinterpret_cast<uint4*>(vdst + j) =
            *reinterpret_cast<const uint4*>(rowp + (size_t)(nh + nkv) * hd + j);
      }
    }
  }
}

// ----------------------------------------------------------------------------- silu(gate) * up
// gu[t] holds gate and up interleaved (gate_0, up_0, gate_1, up_1, ...), as the joined product of
// row-interleaved weights writes them; out[t, i] = gate * 1/(1+exp(-gate)) * up in fp32.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, size_t total) {
  pdl_trigger();
  pdl_wait();
  // two 16-byte loads of (gate, up) pairs and one 16-byte store a thread and pass: 8 pairs of
  // bf16, 4 pairs of fp32
  constexpr int PAIRS = 32 / (2 * (int)sizeof(T));
  const size_t nvec = total / PAIRS;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec;
       i += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw0 = reinterpret_cast<const uint4*>(gu)[2 * i];
    const uint4 raw1 = reinterpret_cast<const uint4*>(gu)[2 * i + 1];
    T in[2 * PAIRS];
    *reinterpret_cast<uint4*>(in) = raw0;
    *reinterpret_cast<uint4*>(in + PAIRS) = raw1;
    T res[PAIRS];
#pragma unroll
    for (int k = 0; k < PAIRS; ++k) {
      const float g = to_f32(in[2 * k]), u = to_f32(in[2 * k + 1]);
      res[k] = from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
    }
    reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(res);
  }
  for (size_t i = nvec * PAIRS + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const float g = to_f32(gu[2 * i]), u = to_f32(gu[2 * i + 1]);
    out[i] = from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
  }
}

template <typename XT, typename T, typename G>
int launch_add_rmsnorm(const void* x, const void* delta, const void* gamma, const int* rows,
                       void* sum_out, void* normed, int R, int H, float eps, cudaStream_t st) {
  // rows of whole octets at 16-byte aligned addresses: the register-resident kernel
  const bool aligned = H % 8 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)delta % 16 == 0) &&
                       ((uintptr_t)gamma % 16 == 0) && ((uintptr_t)sum_out % 16 == 0) &&
                       ((uintptr_t)normed % 16 == 0);
  if (aligned && H <= 8 * 4 * 256) {
    const int noct = H / 8;
    const int opt = noct <= 256 ? 1 : noct <= 512 ? 2 : 4;
    const int threads = ((noct + opt - 1) / opt + 31) / 32 * 32;
#define GF_VEC(OPT)                                                                              \
  return launch_kernel(add_rmsnorm_vec_kernel<XT, T, G, OPT>, dim3(R), dim3(threads), 0, st,      \
                       (const XT*)x, (const T*)delta, (const G*)gamma, rows, (float*)sum_out,     \
                       (T*)normed, H, eps)
    if (opt == 1) GF_VEC(1);
    if (opt == 2) GF_VEC(2);
    GF_VEC(4);
#undef GF_VEC
  }
  const size_t smem = (size_t)2 * H * sizeof(float);
  auto k = add_rmsnorm_kernel<XT, T, G>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
  return launch_kernel(k, dim3(R), dim3(threads), smem, st, (const XT*)x, (const T*)delta,
                       (const G*)gamma, rows, (float*)sum_out, (T*)normed, H, eps);
}

}  // namespace gf

using namespace gf;

GF_DEFINE_PDL_SWITCH

GF_EXPORT int gf_embedding(const int* ids, const void* w, void* out, int T, int H, int dtype,
                           void* stream) {
  if (T <= 0) return 0;
  const size_t row_bytes = (size_t)H * (dtype == GF_F32 ? 4 : 2);
  auto st = (cudaStream_t)stream;
  const bool al16 = row_bytes % 16 == 0 && ((uintptr_t)w % 16 == 0) && ((uintptr_t)out % 16 == 0);
  if (al16)
    return launch_kernel(embedding_kernel<uint4>, dim3(T), dim3(128), 0, st, ids, (const uint4*)w,
                         (uint4*)out, (int)(row_bytes / 16));
  if (dtype == GF_F32)
    return launch_kernel(embedding_kernel<float>, dim3(T), dim3(128), 0, st, ids, (const float*)w,
                         (float*)out, H);
  return launch_kernel(embedding_kernel<uint16_t>, dim3(T), dim3(128), 0, st, ids,
                       (const uint16_t*)w, (uint16_t*)out, H);
}

// x_dtype: type of x (fp32 residual stream, or the activation type); dtype: activation type of
// delta and normed; sum_out (nullable) is fp32.
GF_EXPORT int gf_add_rmsnorm(const void* x, int x_dtype, const void* delta, const void* gamma,
                             int gamma_dtype, float eps, const int* rows, void* sum_out,
                             void* normed, int R, int H, int dtype, void* stream) {
  if (R <= 0) return 0;
  auto st = (cudaStream_t)stream;
  using bf = __nv_bfloat16;
#define GF_GO(XT, T, G) \
  return launch_add_rmsnorm<XT, T, G>(x, delta, gamma, rows, sum_out, normed, R, H, eps, st)
  if (dtype == GF_F32) {
    if (gamma_dtype != GF_F32 || x_dtype != GF_F32) return -2;
    GF_GO(float, float, float);
  }
  if (x_dtype == GF_F32) {
    if (gamma_dtype == GF_F32) GF_GO(float, bf, float);
    GF_GO(float, bf, bf);
  }
  if (gamma_dtype == GF_F32) GF_GO(bf, bf, float);
  GF_GO(bf, bf, bf);
#undef GF_GO
}

GF_EXPORT int gf_rope_kv_write(void* qkv, int row_stride, const float* table, int rot,
                               const int* positions, const int* slot_mapping, void* kpages,
                               void* vpages, int T, int nh, int nkv, int hd, int dtype,
                               void* stream) {
  if (T <= 0) return 0;
  auto st = (cudaStream_t)stream;
  if (!table) rot = 0;
  const int vec = dtype == GF_F32 ? 4 : 8;
  const size_t esz = dtype == GF_F32 ? 4 : 2;
  const bool can_vec = (rot / 2) % vec == 0 && hd % vec == 0 && row_stride % vec == 0 &&
                       ((uintptr_t)qkv % 16 == 0) && ((uintptr_t)kpages % 16 == 0) &&
                       ((uintptr_t)vpages % 16 == 0) && ((size_t)nkv * hd * esz) % 16 == 0;
  if (can_vec) {
    int work = (nh + nkv) * (rot / 2 / vec) + nkv * ((hd - rot) / vec) + nkv * hd / vec;
    int threads = (work + 31) / 32 * 32;
    threads = threads < 32 ? 32 : threads > 256 ? 256 : threads;
    if (dtype == GF_F32)
      return launch_kernel(rope_kv_write_vec_kernel<float>, dim3(T), dim3(threads), 0, st,
                           (float*)qkv, row_stride, table, rot, positions, slot_mapping,
                           (float*)kpages, (float*)vpages, nh, nkv, hd);
    return launch_kernel(rope_kv_write_vec_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, st,
                         (__nv_bfloat16*)qkv, row_stride, table, rot, positions, slot_mapping,
                         (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, nh, nkv, hd);
  }
  int work = (nh + nkv) * (rot / 2);
  if (nkv * hd > work) work = nkv * hd;
  int threads = (work + 31) / 32 * 32;
  threads = threads < 32 ? 32 : threads > 1024 ? 1024 : threads;
  if (dtype == GF_F32)
    return launch_kernel(rope_kv_write_kernel<float>, dim3(T), dim3(threads), 0, st, (float*)qkv,
                         row_stride, table, rot, positions, slot_mapping, (float*)kpages,
                         (float*)vpages, nh, nkv, hd);
  return launch_kernel(rope_kv_write_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, st,
                       (__nv_bfloat16*)qkv, row_stride, table, rot, positions, slot_mapping,
                       (__nv_bfloat16*)kpages, (__nv_bfloat16*)vpages, nh, nkv, hd);
}

GF_EXPORT int gf_silu_mul(const void* gu, void* out, int T, int I, int dtype, void* stream) {
  const size_t total = (size_t)T * I;
  if (total == 0) return 0;
  auto st = (cudaStream_t)stream;
  const size_t want = (total / 4 + 255) / 256 + 1;
  const int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == GF_F32)
    return launch_kernel(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, st, (const float*)gu,
                         (float*)out, total);
  return launch_kernel(silu_mul_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, st,
                       (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total);
}
