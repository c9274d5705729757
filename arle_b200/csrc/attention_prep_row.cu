// Preparation of queries and keys for an attention whose q/k norm runs over the whole
// projected row (all heads at once) and whose values may be the keys as projected.
//
// Input row t of qk: [q heads (nq * hd) | k heads (nkv * hd) | ...] (row stride given).
// One block per token:
//   q: x <- x * q_weight[e] * rsqrt(mean over all nq*hd elements of x^2 + eps) (if q_weight),
//      rotate, store in place;
//   k: the same over the nkv*hd elements with k_weight, rotate, store into k_cache at the
//      token's slot;
//   v: with values_are_keys the row of k as projected (before norm and rotation) goes into
//      v_cache unchanged; otherwise the v heads that follow the k heads in the row do.
// Rotation, within the first rotary_dim elements of each head: pairing 0 turns element i with
// i + rotary_dim/2 ("half split"), pairing 1 turns element 2i with 2i + 1 ("interleaved"); the
// pair (u, v) becomes (u cos a - v sin a, v cos a + u sin a) with a = position * inv_freq[i],
// in float32 (sincosf), or with the cosines and sines of a table [T][rotary_dim/2] of (cos, sin) that was filled the
// same way once for the step (the same bits).  Norm statistics and products are float32.
// Cache layout: [page][kv_head][slot_in_page][head_dim]; slot_mapping[t] < 0: no store.
#include "common.cuh"
using namespace arle;

template <typename T>
__global__ void attention_prep_row_kernel(T* __restrict__ qk, int row_stride, const int* __restrict__ positions,
                                          const int* __restrict__ slot_mapping, const float* __restrict__ q_weight,
                                          const float* __restrict__ k_weight, float eps,
                                          const float* __restrict__ inv_freq, const float2* __restrict__ angles,
                                          int rotary_dim, int pairing, int values_are_keys, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          int nq, int nkv, int hd, int page_size, int vec8) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float row[];                 // (nq + nkv) * hd floats: x * weight, still without the row's factor
  __shared__ float red[2][33];
  const int t = blockIdx.x;
  const int nqe = nq * hd, nke = nkv * hd;
  T* src = qk + (size_t)t * row_stride;
  // everything the block needs from memory is asked for before the first use
  const int slot = nkv > 0 ? slot_mapping[t] : -1;
  const float pos = (float)positions[t];
  float sq = 0.f, sk = 0.f;
  if (sizeof(T) == 2 && vec8) {                  // bfloat16 rows on 16-byte boundaries, q's and k's widths multiples of 8
    for (int e = threadIdx.x * 8; e < nqe + nke; e += blockDim.x * 8) {
      const uint4 u = *reinterpret_cast<const uint4*>(src + e);
      const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
      const float* wt = e < nqe ? q_weight : k_weight;
      const float* wp = wt ? wt + (e < nqe ? e : e - nqe) : nullptr;
      float s = 0.f, xw[8];
      float4 w0 = make_float4(1.f, 1.f, 1.f, 1.f), w1 = w0;
      if (wp) w0 = *reinterpret_cast<const float4*>(wp), w1 = *reinterpret_cast<const float4*>(wp + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a = __low2float(h2[i]), b = __high2float(h2[i]);
        xw[2 * i] = a * wv[2 * i];
        xw[2 * i + 1] = b * wv[2 * i + 1];
        s += a * a + b * b;
      }
      *reinterpret_cast<float4*>(row + e) = make_float4(xw[0], xw[1], xw[2], xw[3]);
      *reinterpret_cast<float4*>(row + e + 4) = make_float4(xw[4], xw[5], xw[6], xw[7]);
      if (e < nqe) sq += s; else sk += s;
    }
  } else {
    for (int e = threadIdx.x; e < nqe + nke; e += blockDim.x) {
      const float x = to_f32(src[e]);
      const float* wt = e < nqe ? q_weight : k_weight;
      const float w = wt ? wt[e < nqe ? e : e - nqe] : 1.0f;
      row[e] = x * w;
      if (e < nqe) sq += x * x; else sk += x * x;
    }
  }
  {                                              // both sums in one pass over the block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) red[0][warp] = sq, red[1][warp] = sk;
    __syncthreads();                             // also: every row[] entry is written
    if (warp < 2) {
      float v = lane < nwarps ? red[warp][lane] : 0.f;
      v = warp_sum(v);
      if (lane == 0) red[warp][32] = v;
    }
    __syncthreads();
    sq = red[0][32], sk = red[1][32];
  }
  const float inv_q = q_weight ? 1.0f / sqrtf(sq / (float)nqe + eps) : 1.0f;
  const float inv_k = k_weight ? 1.0f / sqrtf(sk / (float)(nke > 0 ? nke : 1) + eps) : 1.0f;
  const int page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot - page * page_size : 0;
  const int half = rotary_dim >> 1, hd2 = hd >> 1;
  const float2* ang = angles ? angles + (size_t)t * half : nullptr;
  // a thread takes a pair of elements: the two that turn together, or two neighbours past rotary_dim
  for (int p = threadIdx.x; p < (nq + nkv) * hd2; p += blockDim.x) {
    const int head = p / hd2, d2 = p - head * hd2;
    int e0, e1;
    float o0, o1;
    if (d2 < half) {
      e0 = head * hd + (pairing == 0 ? d2 : 2 * d2);
      e1 = pairing == 0 ? e0 + half : e0 + 1;
      float sn, cs;
      if (ang) {
        const float2 a = ang[d2];
        cs = a.x, sn = a.y;
      } else {
        sincosf(pos * inv_freq[d2], &sn, &cs);
      }
      const float inv = head < nq ? inv_q : inv_k;
      const float x0 = row[e0] * inv, x1 = row[e1] * inv;
      o0 = x0 * cs - x1 * sn;
      o1 = x1 * cs + x0 * sn;
    } else {
      const float inv = head < nq ? inv_q : inv_k;
      e0 = head * hd + rotary_dim + 2 * (d2 - half);
      e1 = e0 + 1;
      o0 = row[e0] * inv, o1 = row[e1] * inv;
    }
    const bool pair = sizeof(T) == 2 && vec8 && e1 == e0 + 1;      // neighbours: one 4-byte access for both
    if (head < nq) {
      if (pair) {
        *reinterpret_cast<__nv_bfloat162*>(src + e0) = __floats2bfloat162_rn(o0, o1);
      } else {
        src[e0] = from_f32<T>(o0);
        src[e1] = from_f32<T>(o1);
      }
    } else if (slot >= 0) {
      const size_t base = (((size_t)page * nkv + (head - nq)) * page_size + off) * hd - (size_t)head * hd;
      const T* vsrc = values_are_keys ? src : src + nke;
      if (pair) {
        *reinterpret_cast<__nv_bfloat162*>(k_cache + base + e0) = __floats2bfloat162_rn(o0, o1);
        *reinterpret_cast<uint32_t*>(v_cache + base + e0) = *reinterpret_cast<const uint32_t*>(vsrc + e0);
      } else {
        k_cache[base + e0] = from_f32<T>(o0);
        k_cache[base + e1] = from_f32<T>(o1);
        v_cache[base + e0] = vsrc[e0];
        v_cache[base + e1] = vsrc[e1];
      }
    }
  }
}

ARLE_API int arle_attention_prep_row(void* qk, int dtype, int row_stride, const int* positions, const int* slot_mapping,
                                     const float* q_weight, const float* k_weight, float eps, const float* inv_freq,
                                     const float* angles, int rotary_dim, int pairing, int values_are_keys, void* k_cache, void* v_cache, int nq,
                                     int nkv, int hd, int page_size, int num_tokens, cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (hd & 1) return ARLE_E_UNSUPPORTED;
  if (hd <= 0 || nq <= 0 || nkv < 0 || page_size <= 0 || rotary_dim < 0 || rotary_dim > hd || (rotary_dim & 1)) return ARLE_E_BADARG;
  if (pairing != 0 && pairing != 1) return ARLE_E_BADARG;
  if (rotary_dim > 0 && !inv_freq) return ARLE_E_BADARG;
  if (nkv > 0 && (!slot_mapping || !k_cache || !v_cache)) return ARLE_E_BADARG;
  const size_t smem = (size_t)(nq + nkv) * hd * sizeof(float);
  if (smem > 200 * 1024) return ARLE_E_UNSUPPORTED;
  const int n = (nq + nkv) * hd;
  const int threads = n >= 512 ? 256 : 128;
  // wide accesses: every row, head and cache entry starts on a 16-byte boundary (even head sizes keep pairs on 4)
  const int vec8 = dtype == 1 && (nq * hd) % 8 == 0 && (nkv * hd) % 8 == 0 && row_stride % 8 == 0 && ((uintptr_t)qk % 16) == 0 &&
                   ((uintptr_t)k_cache % 16) == 0 && ((uintptr_t)v_cache % 16) == 0 && ((uintptr_t)q_weight % 16) == 0 &&
                   ((uintptr_t)k_weight % 16) == 0;
  if (dtype == 0) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(attention_prep_row_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(attention_prep_row_kernel<float>, dim3(num_tokens), dim3(threads), smem, s, 1, (float*)qk, row_stride, positions,
                  slot_mapping, q_weight, k_weight, eps, inv_freq, (const float2*)angles, rotary_dim, pairing, values_are_keys, (float*)k_cache,
                  (float*)v_cache, nq, nkv, hd, page_size, vec8);
  } else if (dtype == 1) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(attention_prep_row_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(attention_prep_row_kernel<__nv_bfloat16>, dim3(num_tokens), dim3(threads), smem, s, 1, (__nv_bfloat16*)qk,
                  row_stride, positions, slot_mapping, q_weight, k_weight, eps, inv_freq, (const float2*)angles, rotary_dim, pairing,
                  values_are_keys,
                  (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, nq, nkv, hd, page_size, vec8);
  } else {
    return ARLE_E_BADARG;
  }
  return launch_status();
}
