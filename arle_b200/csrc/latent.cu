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
//  * latent_attention_mma (bfloat16, rank 64 / 128 / 256 / 512, rotated part a multiple of 16): the same attention on the
//    tensor cores.  Since every head reads the same records, the heads of a token are the rows of the products: a block
//    takes one token, sixteen heads and a share of its keys; a tile of 64 records comes in by cp.async; Q . K^T (16 x 64,
//    the four warps a quarter of the keys each) and P . V (16 x rank, the warps a quarter of the columns each, V being the
//    record's first `rank` columns of the same tile) are mma.sync with float32 sums, the softmax in float32 between them.
//    With few tokens in the step (decoding) a token's keys are shared out among several blocks whose parts
//    latent_merge adds up, so that the machine is filled.
#include "common.cuh"
#include "mma_utils.cuh"
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

constexpr int kMmaTile = 64, kPPitch = 72;

template <int R64>
__global__ void __launch_bounds__(128) latent_attention_mma_kernel(
    const __nv_bfloat16* __restrict__ q_abs, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ row_of_token,
    const int* __restrict__ block_table, int bt_stride, int H, int kd, int page_size, float scale, int window, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int rank = 64 * R64;
  extern __shared__ __align__(16) unsigned char smraw[];
  const int pitch = kd + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smraw);          // [16][pitch]
  __nv_bfloat16* Ks = Qs + 16 * pitch;                                  // [64][pitch]
  __nv_bfloat16* Ps = Ks + kMmaTile * pitch;                            // [16][72]
  float* red = reinterpret_cast<float*>(Ps + 16 * kPPitch);             // [4][16]
  const int t = blockIdx.x, h0 = blockIdx.y * 16, sp = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)row_of_token[t] * bt_stride;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int ntiles = (pos - lo) / kMmaTile + 1;
  const int tps = (ntiles + splits - 1) / splits;
  const int tile_beg = sp * tps, tile_end = min(ntiles, tile_beg + tps);
  const int chunks = kd >> 3;

  for (int idx = tid; idx < 16 * chunks; idx += 128) {
    const int r = idx / chunks, c = (idx - r * chunks) * 8;
    if (h0 + r < H)
      cp_async16(smem_u32(Qs + r * pitch + c), q_abs + ((size_t)t * H + h0 + r) * kd + c, 16);
    else
      *reinterpret_cast<uint4*>(Qs + r * pitch + c) = make_uint4(0, 0, 0, 0);
  }
  float o[2 * R64][4];
#pragma unroll
  for (int i = 0; i < 2 * R64; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  const int cbase = warp * 16 * R64;

  for (int tile = tile_beg; tile < tile_end; ++tile) {
    const int j0 = lo + tile * kMmaTile;
    for (int idx = tid; idx < kMmaTile * chunks; idx += 128) {
      const int r = idx / chunks, c = (idx - r * chunks) * 8;
      const int j = j0 + r;
      const bool ok = j <= pos;
      const __nv_bfloat16* src = ok ? cache + ((size_t)bt[j / page_size] * page_size + j % page_size) * kd + c : cache;
      cp_async16(smem_u32(Ks + r * pitch + c), src, ok ? 16 : 0);
    }
    cp_commit();
    cp_wait<0>();
    __syncthreads();
    float s[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
    for (int kk = 0; kk < (kd >> 4); ++kk) {
      uint32_t a[4], b0, b1, b2, b3;
      ldsm_x4(smem_u32(Qs + (lane & 15) * pitch + kk * 16 + (lane >> 4) * 8), a[0], a[1], a[2], a[3]);
      ldsm_x4(smem_u32(Ks + (warp * 16 + (lane >> 4) * 8 + (lane & 7)) * pitch + kk * 16 + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
      mma_bf16(s[0], a, b0, b1);
      mma_bf16(s[1], a, b2, b3);
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int j = j0 + warp * 16 + n * 8 + 2 * t4 + (i & 1);
        s[n][i] = j <= pos ? s[n][i] * scale : -INFINITY;
      }
    float mx0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    float mx1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    if (t4 == 0) {
      red[warp * 16 + g] = mx0;
      red[warp * 16 + g + 8] = mx1;
    }
    __syncthreads();
    const float mn0 = fmaxf(m0, fmaxf(fmaxf(red[g], red[16 + g]), fmaxf(red[32 + g], red[48 + g])));
    const float mn1 = fmaxf(m1, fmaxf(fmaxf(red[g + 8], red[24 + g]), fmaxf(red[40 + g], red[56 + g])));
    const float c0 = expf(m0 - mn0), c1 = expf(m1 - mn1);        // the tile's first key is visible, so mn is finite
    float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0 = expf(s[n][0] - mn0), p1 = expf(s[n][1] - mn0), p2 = expf(s[n][2] - mn1), p3 = expf(s[n][3] - mn1);
      ps0 += p0 + p1;
      ps1 += p2 + p3;
      const int col = warp * 16 + n * 8 + 2 * t4;
      *reinterpret_cast<uint32_t*>(Ps + g * kPPitch + col) = pack_bf16(p0, p1);
      *reinterpret_cast<uint32_t*>(Ps + (g + 8) * kPPitch + col) = pack_bf16(p2, p3);
    }
    l0 = l0 * c0 + ps0;
    l1 = l1 * c1 + ps1;
    m0 = mn0;
    m1 = mn1;
#pragma unroll
    for (int i = 0; i < 2 * R64; ++i) {
      o[i][0] *= c0; o[i][1] *= c0; o[i][2] *= c1; o[i][3] *= c1;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kMmaTile / 16; ++kk) {
      uint32_t pa[4];
      ldsm_x4(smem_u32(Ps + (lane & 15) * kPPitch + kk * 16 + (lane >> 4) * 8), pa[0], pa[1], pa[2], pa[3]);
#pragma unroll
      for (int dn = 0; dn < R64; ++dn) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(Ks + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * pitch + cbase + dn * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
        mma_bf16(o[2 * dn], pa, b0, b1);
        mma_bf16(o[2 * dn + 1], pa, b2, b3);
      }
    }
    __syncthreads();
  }
  if (tile_beg >= tile_end) {
    cp_commit();
    cp_wait<0>();
  }
  // the rows' sums: over the four lanes of a row, then over the warps (each saw a quarter of every tile's keys)
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();
  if (t4 == 0) {
    red[warp * 16 + g] = l0;
    red[warp * 16 + g + 8] = l1;
  }
  __syncthreads();
  const float lt0 = red[g] + red[16 + g] + red[32 + g] + red[48 + g];
  const float lt1 = red[g + 8] + red[24 + g] + red[40 + g] + red[56 + g];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int h = h0 + g + half * 8;
    if (h >= H) continue;
    const float lt = half ? lt1 : lt0;
    if (splits == 1) {
      const float inv = 1.0f / lt;
      __nv_bfloat16* op = out + ((size_t)t * H + h) * rank + cbase + 2 * t4;
#pragma unroll
      for (int n = 0; n < 2 * R64; ++n)
        *reinterpret_cast<uint32_t*>(op + n * 8) = pack_bf16(o[n][2 * half] * inv, o[n][2 * half + 1] * inv);
    } else {
      const size_t slot = ((size_t)t * H + h) * splits + sp;
      float* op = part_o + slot * rank + cbase + 2 * t4;
#pragma unroll
      for (int n = 0; n < 2 * R64; ++n) {
        op[n * 8] = o[n][2 * half];
        op[n * 8 + 1] = o[n][2 * half + 1];
      }
      if (warp == 0 && t4 == 0) {
        part_ml[slot * 2] = half ? m1 : m0;
        part_ml[slot * 2 + 1] = lt;
      }
    }
  }
}

// The parts of a (token, head) that several blocks hold: out = sum_s e^(m_s - M) o_s / sum_s e^(m_s - M) l_s, s ascending.
__global__ void latent_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, __nv_bfloat16* __restrict__ out,
                                    int rank, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t th = blockIdx.x;
  const float* ml = part_ml + th * splits * 2;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s)
    if (ml[2 * s + 1] > 0.f) M = fmaxf(M, ml[2 * s]);
  float den = 0.f;
  for (int s = 0; s < splits; ++s)
    if (ml[2 * s + 1] > 0.f) den += expf(ml[2 * s] - M) * ml[2 * s + 1];
  const float inv = 1.0f / den;
  for (int c = threadIdx.x; c < rank; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s)
      if (ml[2 * s + 1] > 0.f) acc = fmaf(expf(ml[2 * s] - M), part_o[(th * splits + s) * rank + c], acc);
    out[th * rank + c] = __float2bfloat16_rn(acc * inv);
  }
}

template <int R64>
static int launch_latent_mma(const void* q_abs, void* out, float* part_o, float* part_ml, const void* cache, const int* positions,
                             const int* row_of_token, const int* block_table, int bt_stride, int H, int kd, int page_size, float scale,
                             int window, int num_tokens, int splits, cudaStream_t s) {
  const size_t smem = (size_t)(16 + kMmaTile) * (kd + 8) * 2 + 16 * kPPitch * 2 + 64 * sizeof(float);
  if (smem > 220 * 1024) return ARLE_E_UNSUPPORTED;
  cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<R64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(num_tokens, (H + 15) / 16, splits);
  launch_kernel(latent_attention_mma_kernel<R64>, dim3(grid), dim3(128), smem, s, 1, (const __nv_bfloat16*)q_abs, (__nv_bfloat16*)out,
                part_o, part_ml, (const __nv_bfloat16*)cache, positions, row_of_token, block_table, bt_stride, H, kd, page_size, scale,
                window, splits);
  if (splits > 1)
    launch_kernel(latent_merge_kernel, dim3(num_tokens * H), dim3(64 * R64 >= 256 ? 128 : 64), 0, s, 1, (const float*)part_o,
                  (const float*)part_ml, (__nv_bfloat16*)out, 64 * R64, splits);
  return launch_status();
}

// The tensor-core form: bfloat16, rank 64 / 128 / 256 / 512, kd - rank a multiple of 16.  splits > 1 needs part_o float32
// [T * H * splits * rank] and part_ml float32 [T * H * splits * 2].
ARLE_API int arle_latent_attention_mma(const void* q_abs, void* out, float* part_o, float* part_ml, const void* cache,
                                       const int* positions, const int* row_of_token, const int* block_table, int bt_stride, int H,
                                       int rank, int kd, int page_size, float scale, int window, int num_tokens, int splits,
                                       cudaStream_t s) {
  if (num_tokens <= 0) return 0;
  if (H <= 0 || kd < rank || (kd - rank) % 16 || page_size <= 0 || splits < 1 || splits > 65535 || (H + 15) / 16 > 65535 ||
      (splits > 1 && (!part_o || !part_ml)))
    return ARLE_E_BADARG;
#define ARLE_LAT(R) \
  return launch_latent_mma<R>(q_abs, out, part_o, part_ml, cache, positions, row_of_token, block_table, bt_stride, H, kd, page_size, \
                              scale, window, num_tokens, splits, s)
  if (rank == 64) ARLE_LAT(1);
  if (rank == 128) ARLE_LAT(2);
  if (rank == 256) ARLE_LAT(4);
  if (rank == 512) ARLE_LAT(8);
#undef ARLE_LAT
  return ARLE_E_UNSUPPORTED;
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
