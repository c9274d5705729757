// Small elementwise kernels around mixers that stand side by side.
//
//  * head_gate: out[t, h, :] = x[t, h, :] * sigmoid(g[t, h]) * scale, one gate number per (token, head)
//    taken from a wider row (the packed input projection; no gate pointer: a scaled copy); float32 arithmetic, rounded once.  The
//    output may be a slice of a wider buffer (row stride given).
//  * weighted_sum: out = a * x + b * y in float32, rounded once (the outputs of two mixers that were
//    projected separately).
//  * logit_cap: y <- cap * tanh(y / cap), in place on float32 logits.
#include "common.cuh"
using namespace arle;

template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ g, int g_stride, float scale,
                                 T* __restrict__ out, int out_stride, int heads, int hd, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  const int width = heads * hd;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width;
    const int e = (int)(idx - t * width);
    const float s = g ? 1.0f / (1.0f + expf(-to_f32(g[t * g_stride + e / hd]))) : 1.0f;
    out[t * out_stride + e] = from_f32<T>(to_f32(x[t * x_stride + e]) * (s * scale));
  }
}

// Eight consecutive elements (of one head) per thread: bfloat16 rows whose head size is a multiple of 8 and whose
// rows start on 16-byte boundaries.
__global__ void head_gate_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, int x_stride, const __nv_bfloat16* __restrict__ g,
                                          int g_stride, float scale, __nv_bfloat16* __restrict__ out, int out_stride, int heads,
                                          int hd, size_t total8) {
  pdl_launch_dependents();
  pdl_wait();
  const int w8 = heads * hd / 8;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / w8;
    const int e = (int)(idx - t * w8) * 8;
    const float s = (g ? 1.0f / (1.0f + expf(-__bfloat162float(g[t * g_stride + e / hd]))) : 1.0f) * scale;
    const uint4 u = *reinterpret_cast<const uint4*>(x + t * x_stride + e);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 o4;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
    for (int i = 0; i < 4; ++i) o2[i] = __floats2bfloat162_rn(__low2float(h[i]) * s, __high2float(h[i]) * s);
    *reinterpret_cast<uint4*>(out + t * out_stride + e) = o4;
  }
}

template <typename T>
__global__ void weighted_sum_kernel(const T* __restrict__ x, float a, const T* __restrict__ y, float b, T* __restrict__ out,
                                    size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    out[idx] = from_f32<T>(a * to_f32(x[idx]) + b * to_f32(y[idx]));
}

__global__ void logit_cap_kernel(float* __restrict__ y, float cap, float inv_cap, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x)
    y[idx] = cap * tanhf(y[idx] * inv_cap);
}

static int blocks_for(size_t total, int threads) {
  size_t b = (total + threads - 1) / threads;
  if (b > 148 * 32) b = 148 * 32;
  return (int)b;
}

ARLE_API int arle_head_gate(const void* x, int x_stride, const void* g, int g_stride, float scale, void* out, int out_stride,
                            int dtype, int num_tokens, int heads, int hd, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (heads <= 0 || hd <= 0) return ARLE_E_BADARG;
  const size_t total = (size_t)num_tokens * heads * hd;
  const int threads = 256;
  if (dtype == 1 && hd % 8 == 0 && x_stride % 8 == 0 && out_stride % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0) {
    launch_kernel(head_gate_bf16_vec_kernel, dim3(blocks_for(total / 8, threads)), dim3(threads), 0, s, 1, (const __nv_bfloat16*)x,
                  x_stride, (const __nv_bfloat16*)g, g_stride, scale, (__nv_bfloat16*)out, out_stride, heads, hd, total / 8);
    return launch_status();
  }
  if (dtype == 0)
    launch_kernel(head_gate_kernel<float>, dim3(blocks_for(total, threads)), dim3(threads), 0, s, 1, (const float*)x, x_stride,
                  (const float*)g, g_stride, scale, (float*)out, out_stride, heads, hd, total);
  else if (dtype == 1)
    launch_kernel(head_gate_kernel<__nv_bfloat16>, dim3(blocks_for(total, threads)), dim3(threads), 0, s, 1, (const __nv_bfloat16*)x,
                  x_stride, (const __nv_bfloat16*)g, g_stride, scale, (__nv_bfloat16*)out, out_stride, heads, hd, total);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

ARLE_API int arle_weighted_sum(const void* x, float a, const void* y, float b, void* out, int dtype, long long total,
                               cudaStream_t s) {
  if (total <= 0) return 0;
  const int threads = 256;
  if (dtype == 0)
    launch_kernel(weighted_sum_kernel<float>, dim3(blocks_for((size_t)total, threads)), dim3(threads), 0, s, 1, (const float*)x, a,
                  (const float*)y, b, (float*)out, (size_t)total);
  else if (dtype == 1)
    launch_kernel(weighted_sum_kernel<__nv_bfloat16>, dim3(blocks_for((size_t)total, threads)), dim3(threads), 0, s, 1,
                  (const __nv_bfloat16*)x, a, (const __nv_bfloat16*)y, b, (__nv_bfloat16*)out, (size_t)total);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

ARLE_API int arle_logit_cap(float* y, float cap, long long total, cudaStream_t s) {
  if (total <= 0) return 0;
  if (!(cap > 0.f)) return ARLE_E_BADARG;
  launch_kernel(logit_cap_kernel, dim3(blocks_for((size_t)total, 256)), dim3(256), 0, s, 1, y, cap, 1.0f / cap, (size_t)total);
  return launch_status();
}
