// Gated linear attention: a recurrent mixer with a matrix state per head,
//
//     S_t = diag(alpha_t) S_(t-1) + k_t v_t^T          S: [dim, vdim], float32, one per (request, head)
//     o_t = S_t^T q_t
//
// with a decay alpha_t in (0, 1) per key channel.  Three kernels:
//
//  * gla_decay: alpha[t, c] = sigmoid(z)^(1/tau), z = b[c] + sum_r low[t, r] * w2[c, r], the second
//    half of a low-rank gate (low = W_a1 x comes from the packed input projection).  Evaluated as
//    exp(-softplus(-z) / tau) in float32.
//  * gla_scan: the recurrence over this step's tokens of every request row, from the state that the
//    request's slot holds, which is left updated.  Float32 throughout; q, k, v are read in the
//    activation type.  One block per (columns of vdim, head, row); a thread keeps 16 consecutive key
//    channels of one column of S in registers (lanes_per_col consecutive lanes share a column; the state
//    is stored [vdim][dim] so that these are 64 contiguous bytes), the step's
//    q, k, alpha and v are staged in shared memory a chunk of tokens at a time, and o_t[j] is the sum
//    over the column's lanes.  The order of every sum depends on (dim, vdim) only: a token's result
//    does not depend on how the prompt was cut or on what else is in the batch.
//  * gla_out: per head, o / sqrt(mean(o^2) + eps) * weight (shared by the heads), times silu(gate),
//    times a constant, rounded once into the activation type (a row of a wider buffer may be given).
#include "common.cuh"
using namespace arle;

constexpr int kScanThreads = 128;
constexpr int kScanDpt = 16;                     // key channels per thread

template <typename T>
__global__ void gla_decay_kernel(const T* __restrict__ low, int low_stride, const float* __restrict__ w2,
                                 const float* __restrict__ bias, float inv_tau, float* __restrict__ alpha, int channels,
                                 int rank) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float lo_s[];                // rank floats
  const int t = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) lo_s[r] = to_f32(low[(size_t)t * low_stride + r]);
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < channels; c += gridDim.y * blockDim.x) {
    const float* wr = w2 + (size_t)c * rank;
    float z = 0.f;
    for (int r = 0; r < rank; ++r) z = fmaf(lo_s[r], wr[r], z);
    if (bias) z += bias[c];
    const float y = -z;                          // softplus(y) = log(1 + e^y), the stable way
    const float sp = y > 0.f ? y + log1pf(expf(-y)) : log1pf(expf(y));
    alpha[(size_t)t * channels + c] = expf(-sp * inv_tau);
  }
}

template <typename T>
__global__ void __launch_bounds__(kScanThreads) gla_scan_kernel(
    const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int in_stride,
    const float* __restrict__ alpha, float* __restrict__ state, const int* __restrict__ q_indptr,
    const int* __restrict__ state_slots, float* __restrict__ out, int heads, int dim, int vdim, int lpc, int chunk,
    float q_scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int cols = kScanThreads / lpc;
  const int dpad = (kScanDpt + 1) * lpc;         // channel c sits at c + c / 16: lanes of a column hit different banks
  float* qs = sm;                                // [chunk][dpad]
  float* ks = qs + (size_t)chunk * dpad;
  float* as = ks + (size_t)chunk * dpad;
  float* vs = as + (size_t)chunk * dpad;         // [chunk][cols]
  const int r = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * cols;
  const int l = threadIdx.x & (lpc - 1), jl = threadIdx.x / lpc;
  const int j = j0 + jl;
  const bool col_ok = j < vdim;
  const int t_begin = q_indptr[r], t_end = q_indptr[r + 1];
  // the state of a head is kept as [vdim][dim]: a thread's 16 channels of its column are contiguous
  float* S_g = state + (((size_t)state_slots[r] * heads + h) * vdim + (col_ok ? j : 0)) * dim + l * kScanDpt;
  const bool vec = (dim & 3) == 0;
  float S[kScanDpt];
#pragma unroll
  for (int i = 0; i < kScanDpt; i += 4) {
    const int c = l * kScanDpt + i;
    if (vec) {
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
      if (col_ok && c < dim) u = *reinterpret_cast<const float4*>(S_g + i);
      S[i] = u.x, S[i + 1] = u.y, S[i + 2] = u.z, S[i + 3] = u.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) S[i + e] = (col_ok && c + e < dim) ? S_g[i + e] : 0.f;
    }
  }
  const size_t hq = (size_t)h * dim, hv = (size_t)h * vdim;
  const int dspan = kScanDpt * lpc;              // dim rounded up; channels past dim hold zeros
  for (int t0 = t_begin; t0 < t_end; t0 += chunk) {
    const int n = min(chunk, t_end - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < n * dspan; idx += kScanThreads) {
      const int tt = idx / dspan, c = idx - tt * dspan;
      const size_t row = (size_t)(t0 + tt);
      const bool ok = c < dim;
      const int at = tt * dpad + c + c / kScanDpt;
      qs[at] = ok ? to_f32(q[row * in_stride + hq + c]) * q_scale : 0.f;
      ks[at] = ok ? to_f32(k[row * in_stride + hq + c]) : 0.f;
      as[at] = ok ? alpha[row * heads * dim + hq + c] : 0.f;
    }
    for (int idx = threadIdx.x; idx < n * cols; idx += kScanThreads) {
      const int tt = idx / cols, c = idx - tt * cols;
      vs[idx] = j0 + c < vdim ? to_f32(v[(size_t)(t0 + tt) * in_stride + hv + j0 + c]) : 0.f;
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float vj = vs[tt * cols + jl];
      const float* qt = qs + tt * dpad + l * (kScanDpt + 1);
      const float* kt = ks + tt * dpad + l * (kScanDpt + 1);
      const float* at = as + tt * dpad + l * (kScanDpt + 1);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < kScanDpt; ++i) {
        S[i] = fmaf(at[i], S[i], kt[i] * vj);
        acc[i & 3] = fmaf(S[i], qt[i], acc[i & 3]);
      }
      float o = (acc[0] + acc[1]) + (acc[2] + acc[3]);
      for (int w = lpc >> 1; w > 0; w >>= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
      if (l == 0 && col_ok) out[(size_t)(t0 + tt) * heads * vdim + hv + j] = o;
    }
  }
#pragma unroll
  for (int i = 0; i < kScanDpt; i += 4) {
    const int c = l * kScanDpt + i;
    if (vec) {
      if (col_ok && c < dim) *reinterpret_cast<float4*>(S_g + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (col_ok && c + e < dim) S_g[i + e] = S[i + e];
    }
  }
}

template <typename T>
__global__ void gla_out_kernel(const float* __restrict__ o, const T* __restrict__ gate, int gate_stride,
                               const float* __restrict__ weight, float eps, float scale, T* __restrict__ out,
                               int out_stride, int heads, int vdim, long long units) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= units) return;
  const long long t = unit / heads;
  const int h = (int)(unit - t * heads);
  const float* src = o + ((size_t)t * heads + h) * vdim;
  float ss = 0.f;
  for (int e = lane; e < vdim; e += 32) ss += src[e] * src[e];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
  for (int e = lane; e < vdim; e += 32) {
    float y = src[e] * inv;
    if (weight) y *= weight[e];
    if (gate) {
      const float g = to_f32(gate[(size_t)t * gate_stride + (size_t)h * vdim + e]);
      y *= g / (1.0f + expf(-g));
    }
    out[(size_t)t * out_stride + (size_t)h * vdim + e] = from_f32<T>(y * scale);
  }
}

ARLE_API int arle_gla_decay(const void* low, int dtype, int low_stride, const float* w2, const float* bias, float tau,
                            float* alpha, int num_tokens, int channels, int rank, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (channels <= 0 || rank <= 0 || !(tau > 0.f) || rank > 8192) return ARLE_E_BADARG;
  const int threads = 256;
  int by = (channels + threads - 1) / threads;
  if (by > 64) by = 64;
  const size_t smem = (size_t)rank * sizeof(float);
  if (dtype == 0)
    launch_kernel(gla_decay_kernel<float>, dim3(num_tokens, by), dim3(threads), smem, s, 1, (const float*)low, low_stride, w2, bias,
                  1.0f / tau, alpha, channels, rank);
  else if (dtype == 1)
    launch_kernel(gla_decay_kernel<__nv_bfloat16>, dim3(num_tokens, by), dim3(threads), smem, s, 1, (const __nv_bfloat16*)low,
                  low_stride, w2, bias, 1.0f / tau, alpha, channels, rank);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

// Lanes that share a column of the state: the least power of two that gives every thread at most 16
// key channels.
static int scan_lanes_per_col(int dim) {
  int lpc = 1;
  while (lpc * kScanDpt < dim) lpc <<= 1;
  return lpc;
}

ARLE_API int arle_gla_scan(const void* q, const void* k, const void* v, int dtype, int in_stride, const float* alpha,
                           float* state, const int* q_indptr, const int* state_slots, float* out, int rows, int heads,
                           int dim, int vdim, float q_scale, int max_q_len, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || max_q_len <= 0) return ARLE_E_BADARG;
  if (dim > 32 * kScanDpt || heads > 65535 || rows > 65535) return ARLE_E_UNSUPPORTED;
  const int lpc = scan_lanes_per_col(dim);
  const int cols = kScanThreads / lpc, dpad = (kScanDpt + 1) * lpc;
  const int per_token = (3 * dpad + cols) * (int)sizeof(float);
  int chunk = (40 * 1024) / per_token;
  if (chunk > 16) chunk = 16;
  if (chunk > max_q_len) chunk = max_q_len;
  if (chunk < 1) chunk = 1;
  const size_t smem = (size_t)chunk * per_token;
  dim3 grid((vdim + cols - 1) / cols, heads, rows);
  if (dtype == 0)
    launch_kernel(gla_scan_kernel<float>, grid, dim3(kScanThreads), smem, s, 1, (const float*)q, (const float*)k, (const float*)v,
                  in_stride, alpha, state, q_indptr, state_slots, out, heads, dim, vdim, lpc, chunk, q_scale);
  else if (dtype == 1)
    launch_kernel(gla_scan_kernel<__nv_bfloat16>, grid, dim3(kScanThreads), smem, s, 1, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, in_stride, alpha, state, q_indptr, state_slots, out, heads, dim,
                  vdim, lpc, chunk, q_scale);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

ARLE_API int arle_gla_out(const float* o, const void* gate, int dtype, int gate_stride, const float* weight, float eps,
                          float scale, void* out, int out_stride, int num_tokens, int heads, int vdim, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (heads <= 0 || vdim <= 0) return ARLE_E_BADARG;
  const long long units = (long long)num_tokens * heads;
  const int warps = 8;
  const long long blocks = (units + warps - 1) / warps;
  if (blocks > 0x7fffffffLL) return ARLE_E_UNSUPPORTED;
  if (dtype == 0)
    launch_kernel(gla_out_kernel<float>, dim3((unsigned)blocks), dim3(warps * 32), 0, s, 1, o, (const float*)gate, gate_stride, weight,
                  eps, scale, (float*)out, out_stride, heads, vdim, units);
  else if (dtype == 1)
    launch_kernel(gla_out_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(warps * 32), 0, s, 1, o, (const __nv_bfloat16*)gate,
                  gate_stride, weight, eps, scale, (__nv_bfloat16*)out, out_stride, heads, vdim, units);
  else
    return ARLE_E_BADARG;
  return launch_status();
}
