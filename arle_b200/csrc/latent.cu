// Attention over a cache of latent vectors: every token keeps ONE record [c | k_rot] of rank + rot elements
// (c: the normed latent all heads' keys and values are linear maps of; k_rot: one rotated key part shared by
// all heads).  With the heads' key maps folded into the queries (q_lat[h] = W_uk[h]^T q_nope[h]) and their
// value maps applied after the weighted sum, head h's score against key j is
//     (q_lat[h] . c_j + q_rot[h] . k_rot_j) * scale
// and its output sum_j p_j c_j, so every head reads the same records: multi-query attention whose keys are
// the whole record and whose values are the record's first `rank` elements.
//
//  * latent_prep: per token, RMSNorm of the latent part with its weight, rotation of the shared key part
//    (element i with i + rot_dims/2, angle position * inv_freq[i] in float32, elements past rot_dims pass),
//    the record's store into the paged cache, and the rotation of every head's rotated query part into the
//    folded queries' last `rot` columns.
//  * latent_attention: one block per (token, group of heads).  A tile of 32 records is staged in shared
//    memory once for all heads of the block; a warp owns one or two heads: lane j scores key j, the softmax
//    runs online per head in float32, then lane d accumulates output elements d, d + 32, ...  Tiles are counted
//    from the first visible key max(0, p - window + 1), so the order of every sum depends on (first key, p)
//    alone: a token's result is the same however the prompt was cut and whatever else is in the batch.
#include "common.cuh"
using namespace arle;

template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ dkv, int dkv_stride,
                                   const int* __restrict__ positions, const int* __restrict__ slot_mapping,
                                   const float* __restrict__ c_weight, float eps, const float* __restrict__ inv_freq,
                                   int rot_dims, T* __restrict__ cache, T* __restrict__ q_abs, int H, int dn, int dr, int rank) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int kd = rank + dr, half = rot_dims >> 1;
  const T* kv = dkv + (size_t)t * dkv_stride;
  if (cache != nullptr) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) {
      const float x = to_f32(kv[c]);
      ss += x * x;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)rank + eps);
    T* dst = cache + (size_t)slot_mapping[t] * kd;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32(kv[c]) * inv * c_weight[c]);
    for (int i = threadIdx.x; i < dr; i += blockDim.x) {
      float o;
      if (i < rot_dims) {
        const int p = i < half ? i : i - half;
        float sn, cs;
        sincosf(pos * inv_freq[p], &sn, &cs);
        const float u = to_f32(kv[rank + p]), v = to_f32(kv[rank + p + half]);
        o = i < half ? u * cs - v * sn : v * cs + u * sn;
      } else {
        o = to_f32(kv[rank + i]);
      }
      dst[rank + i] = from_f32<T>(o);
    }
  }
  for (int idx = threadIdx.x; idx < H * dr; idx += blockDim.x) {
    const int h = idx / dr, i = idx - h * dr;
    const T* qp = q + (size_t)t * q_stride + (size_t)h * (dn + dr) + dn;
    float o;
    if (i < rot_dims) {
      const int p = i < half ? i : i - half;
      float sn, cs;
      sincosf(pos * inv_freq[p], &sn, &cs);
      const float u = to_f32(qp[p]), v = to_f32(qp[p + half]);
      o = i < half ? u * cs - v * sn : v * cs + u * sn;
    } else {
      o = to_f32(qp[i]);
    }
    q_abs[((size_t)t * H + h) * kd + rank + i] = from_f32<T>(o);
  }
}

ARLE_API int arle_latent_prep(const void* q, int q_stride, const void* dkv, int dkv_stride, int dtype, const int* positions,
                              const int* slot_mapping, const float* c_weight, float eps, const float* inv_freq, int rot_dims,
                              void* cache, void* q_abs, int H, int dn, int dr, int rank, int num_tokens, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || dn < 0 || dr < 0 || rank <= 0 || rot_dims < 0 || rot_dims > dr || (rot_dims & 1)) return ARLE_E_BADARG;
  const int threads = 128;
  if (dtype == 0)
    launch_kernel(latent_prep_kernel<float>, dim3(num_tokens), dim3(threads), 0, s, 1, (const float*)q, q_stride, (const float*)dkv,
                  dkv_stride, positions, slot_mapping, c_weight, eps, inv_freq, rot_dims, (float*)cache, (float*)q_abs, H, dn, dr, rank);
  else if (dtype == 1)
    launch_kernel(latent_prep_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), 0, s, 1, (const __nv_bfloat16*)q, q_stride,
                  (const __nv_bfloat16*)dkv, dkv_stride, positions, slot_mapping, c_weight, eps, inv_freq, rot_dims,
                  (__nv_bfloat16*)cache, (__nv_bfloat16*)q_abs, H, dn, dr, rank);
  else
    return ARLE_E_BADARG;
  return launch_status();
}

constexpr int kLatTile = 32;      // records per tile
constexpr int kLatMaxD = 16;      // rank <= 512

template <typename T, int HPW>
__global__ void latent_attention_kernel(const T* __restrict__ q_abs, T* __restrict__ out, const T* __restrict__ cache,
                                        const int* __restrict__ positions, const int* __restrict__ row_of_token,
                                        const int* __restrict__ block_table, int bt_stride, int H, int rank, int kd,
                                        int page_size, float scale, int window) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  const int ks_ld = kd + 1;
  float* ks = sm;                              // [kLatTile][kd + 1]
  float* qs = sm + kLatTile * ks_ld;           // [heads of the block][kd]
  const int t = blockIdx.x;
  const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hb = (blockDim.x >> 5) * HPW;
  const int h0 = blockIdx.y * hb;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)row_of_token[t] * bt_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  for (int idx = threadIdx.x; idx < hb * kd; idx += blockDim.x) {
    const int h = h0 + idx / kd;
    qs[idx] = h < H ? to_f32(q_abs[((size_t)t * H + h) * kd + idx % kd]) * scale : 0.f;
  }
  float m[HPW], l[HPW], acc[HPW][kLatMaxD];
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int d = 0; d < kLatMaxD; ++d) acc[i][d] = 0.f;
  }
  for (int j0 = lo; j0 <= pos; j0 += kLatTile) {
    const int n = min(kLatTile, pos - j0 + 1);
    __syncthreads();
    for (int jj = w; jj < n; jj += (blockDim.x >> 5)) {
      const int j = j0 + jj;
      const T* rec = cache + ((size_t)bt[j / page_size] * page_size + j % page_size) * kd;
      for (int e = lane; e < kd; e += 32) ks[jj * ks_ld + e] = to_f32(rec[e]);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      if (h0 + w * HPW + i >= H) continue;
      const float* qh = qs + (w * HPW + i) * kd;
      float sc = -INFINITY;
      if (lane < n) {
        const float* kr = ks + lane * ks_ld;
        float d = 0.f;
        for (int e = 0; e < kd; ++e) d = fmaf(qh[e], kr[e], d);
        sc = d;
      }
      const float m_new = fmaxf(m[i], warp_max(sc));
      const float p = lane < n ? expf(sc - m_new) : 0.f;
      const float corr = expf(m[i] - m_new);
      l[i] = l[i] * corr + warp_sum(p);
      m[i] = m_new;
#pragma unroll
      for (int d = 0; d < kLatMaxD; ++d) acc[i][d] *= corr;
      for (int jj = 0; jj < n; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const float* vr = ks + jj * ks_ld;
#pragma unroll
        for (int d = 0; d < kLatMaxD; ++d) {
          const int c = lane + 32 * d;
          if (c < rank) acc[i][d] = fmaf(pj, vr[c], acc[i][d]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int h = h0 + w * HPW + i;
    if (h >= H) continue;
    T* op = out + ((size_t)t * H + h) * rank;
    const float inv = 1.0f / l[i];
#pragma unroll
    for (int d = 0; d < kLatMaxD; ++d) {
      const int c = lane + 32 * d;
      if (c < rank) op[c] = from_f32<T>(acc[i][d] * inv);
    }
  }
}

template <typename T, int HPW>
static int launch_latent(const void* q_abs, void* out, const void* cache, const int* positions, const int* row_of_token,
                         const int* block_table, int bt_stride, int H, int rank, int kd, int page_size, float scale, int window,
                         int num_tokens, int warps, cudaStream_t s) {
  const int hb = warps * HPW;
  const size_t smem = ((size_t)kLatTile * (kd + 1) + (size_t)hb * kd) * sizeof(float);
  if (smem > 220 * 1024) return ARLE_E_UNSUPPORTED;
  if (smem > 40 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_kernel<T, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(num_tokens, (H + hb - 1) / hb);
  launch_kernel(latent_attention_kernel<T, HPW>, dim3(grid), dim3(warps * 32), smem, s, 1, (const T*)q_abs, (T*)out, (const T*)cache,
                positions, row_of_token, block_table, bt_stride, H, rank, kd, page_size, scale, window);
  return launch_status();
}

// q_abs [T, H, kd] (folded queries: rank columns, then the rotated part), out [T, H, rank], cache [pages, 1, page_size, kd].
ARLE_API int arle_latent_attention(const void* q_abs, void* out, const void* cache, int dtype, const int* positions,
                                   const int* row_of_token, const int* block_table, int bt_stride, int H, int rank, int kd,
                                   int page_size, float scale, int window, int num_tokens, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || rank <= 0 || kd < rank || page_size <= 0) return ARLE_E_BADARG;
  if (rank > 32 * kLatMaxD || H > 65535 * 8) return ARLE_E_UNSUPPORTED;
  const bool two = H > 8;
  const int warps = two ? 8 : H;
  if (dtype == 0)
    return two ? launch_latent<float, 2>(q_abs, out, cache, positions, row_of_token, block_table, bt_stride, H, rank, kd, page_size,
                                         scale, window, num_tokens, warps, s)
               : launch_latent<float, 1>(q_abs, out, cache, positions, row_of_token, block_table, bt_stride, H, rank, kd, page_size,
                                         scale, window, num_tokens, warps, s);
  if (dtype == 1)
    return two ? launch_latent<__nv_bfloat16, 2>(q_abs, out, cache, positions, row_of_token, block_table, bt_stride, H, rank, kd,
                                                 page_size, scale, window, num_tokens, warps, s)
               : launch_latent<__nv_bfloat16, 1>(q_abs, out, cache, positions, row_of_token, block_table, bt_stride, H, rank, kd,
                                                 page_size, scale, window, num_tokens, warps, s);
  return ARLE_E_BADARG;
}
