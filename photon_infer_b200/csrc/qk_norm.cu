// Per-head RMS norm of queries and keys, rotation of their first dimensions, and the write of keys and values into
// the paged cache, in one pass over the projected row of a token.
//
//   y = x / sqrt(mean(x^2) + eps) [* w]           per head, over its d numbers; w [d] is shared by all heads
//   (y[j], y[j + r/2]) <- (y[j] c - y[j + r/2] s, y[j + r/2] c + y[j] s),  j < r/2, angle = position * inv_freq[j]
//
// r = rot_dims <= d; the other d - r numbers of a head pass unrotated.  Norm and rotation are 32-bit, the angle and its
// sine and cosine 64-bit (a position of a few thousand times a frequency near 1 leaves 1e-4 of an angle's error in
// 32-bit); every result is rounded once, to the type of the attention input and of the cache.  The input row may
// be 32-bit while queries and cache are bfloat16: the projection then hands over its unrounded sums.
// Values are copied (and rounded) into their cache; a value may have another width (dv) than a key (d).
// A slot of -1 stores nothing.
#include "common.cuh"
#include <math.h>

#define QKN_WARPS 4

// Four consecutive elements as one load or store (16 bytes of float, 8 of bfloat16).
__device__ __forceinline__ void qkn_load4(const float* p, float* f) { const float4 r = *reinterpret_cast<const float4*>(p); f[0] = r.x; f[1] = r.y; f[2] = r.z; f[3] = r.w; }
__device__ __forceinline__ void qkn_load4(const bf16* p, float* f) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void qkn_store4(float* p, const float* f) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
__device__ __forceinline__ void qkn_store4(bf16* p, const float* f) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&a);
  r.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}

// VEC: rows are read and written four elements at a time (d and dv multiples of 4, aligned pointers and strides).
template <typename TI, typename TO, bool VEC>
__global__ void __launch_bounds__(QKN_WARPS * 32)
qk_norm_rope_write_kernel(const TI* q, long q_stride, const TI* k, long k_stride, const TI* v, long v_stride,
                          TO* q_out, long qo_stride, const void* __restrict__ q_w, const void* __restrict__ k_w,
                          int w_bf16, float eps, const int* __restrict__ positions,
                          const double* __restrict__ inv_freq, int rot_dims, const int* __restrict__ slot_mapping,
                          TO* __restrict__ k_cache, TO* __restrict__ v_cache, int n_q, int n_kv, int d, int dv,
                          int page_size, long num_slots, int* err) {
  extern __shared__ __align__(16) float qkn_smem[];
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.y;
  const int item = blockIdx.x * QKN_WARPS + warp;
  const int kv_items = k_cache ? n_kv : 0;
  if (item >= n_q + 2 * kv_items) return;
  const int which = item < n_q ? 0 : (item < n_q + kv_items ? 1 : 2);
  const int h = which == 0 ? item : (which == 1 ? item - n_q : item - n_q - kv_items);
  float* xs = qkn_smem + (size_t)warp * d;

  long slot = -1;
  size_t page_at = 0;
  if (which != 0) {
    slot = slot_mapping[t];
    if (slot >= num_slots || slot < -1) {
      if (lane == 0 && which == 1 && h == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, (int)slot, (int)num_slots);
      slot = -1;
    }
    if (slot >= 0) {
      const long page = slot / page_size;
      page_at = ((size_t)page * n_kv + h) * page_size + (size_t)(slot - page * page_size);
    }
  }
  if (which == 2) {
    if (slot >= 0) {
      const TI* vr = v + (size_t)t * v_stride + (size_t)h * dv;
      TO* dst = v_cache + page_at * dv;
      if (VEC) {
        for (int i = lane * 4; i < dv; i += 128) { float f[4]; qkn_load4(vr + i, f); qkn_store4(dst + i, f); }
      } else {
        for (int i = lane; i < dv; i += 32) dst[i] = from_f32<TO>(to_f32(vr[i]));
      }
    }
    return;
  }
  const TI* row = (which == 0 ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)h * d;
  float ss = 0.f;
  if (VEC) {
    for (int i = lane * 4; i < d; i += 128) {
      float f[4];
      qkn_load4(row + i, f);
      *reinterpret_cast<float4*>(xs + i) = make_float4(f[0], f[1], f[2], f[3]);
      ss += (f[0] * f[0] + f[1] * f[1]) + (f[2] * f[2] + f[3] * f[3]);
    }
  } else {
    for (int i = lane; i < d; i += 32) { const float x = to_f32(row[i]); xs[i] = x; ss += x * x; }
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / (float)d + eps);
  const void* w = which == 0 ? q_w : k_w;
  __syncwarp();
  for (int i = lane; i < d; i += 32) xs[i] = w ? xs[i] * inv * load_w(w, w_bf16, i) : xs[i] * inv;
  __syncwarp();
  if (rot_dims > 0) {
    const int half = rot_dims >> 1;
    const double pos = (double)positions[t];
    for (int j = lane; j < half; j += 32) {
      double sn, cs;
      sincos(pos * inv_freq[j], &sn, &cs);
      const float c = (float)cs, s = (float)sn;
      const float a = xs[j], b = xs[j + half];
      xs[j] = a * c - b * s;
      xs[j + half] = b * c + a * s;
    }
    __syncwarp();
  }
  TO* dst = nullptr;
  if (which == 0) dst = q_out + (size_t)t * qo_stride + (size_t)h * d;
  else if (slot >= 0) dst = k_cache + page_at * d;
  if (dst != nullptr) {
    if (VEC) {
      for (int i = lane * 4; i < d; i += 128) qkn_store4(dst + i, xs + i);
    } else {
      for (int i = lane; i < d; i += 32) dst[i] = from_f32<TO>(xs[i]);
    }
  }
}

// q [T, n_q * d], k [T, n_kv * d], v [T, n_kv * dv] of in_dtype, each with its own row stride in elements (sections of
// one fused row as a rule).  q_out [T, n_q * d] of out_dtype (row stride qo_stride).  q_w, k_w: norm weights [d] of
// w_dtype, or null for a norm without a weight.  inv_freq: double [rot_dims / 2], null or rot_dims 0: no rotation.
// k_cache [pages, n_kv, page_size, d], v_cache [pages, n_kv, page_size, dv] of out_dtype; both null: nothing is stored
// (an entry that reads another entry's pages), and k and v are not read.
PHOTON_API int photon_qk_norm_rope_write(const void* q, long q_stride, const void* k, long k_stride, const void* v,
                                         long v_stride, int in_dtype, void* q_out, long qo_stride, int out_dtype,
                                         const void* q_w, const void* k_w, int w_dtype, float eps, const int* positions,
                                         const double* inv_freq, int rot_dims, const int* slot_mapping, void* k_cache,
                                         void* v_cache, int T, int n_q, int n_kv, int d, int dv, int page_size,
                                         long num_slots, int* err, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (d <= 0 || dv <= 0 || n_q <= 0 || n_kv <= 0 || rot_dims < 0 || (rot_dims & 1) || rot_dims > d) return PHOTON_ERR_ARGUMENT;
  if ((k_cache == nullptr) != (v_cache == nullptr)) return PHOTON_ERR_ARGUMENT;
  if (T > 65535 || d > 8192) return PHOTON_ERR_UNSUPPORTED;
  if (inv_freq == nullptr) rot_dims = 0;
  const int items = n_q + (k_cache ? 2 * n_kv : 0);
  dim3 grid((items + QKN_WARPS - 1) / QKN_WARPS, T);
  const size_t smem = (size_t)QKN_WARPS * d * sizeof(float);
  const int wb = (w_dtype == PHOTON_BF16);
  const uintptr_t ia = in_dtype == PHOTON_F32 ? 16 : 8, oa = out_dtype == PHOTON_F32 ? 16 : 8;   // bytes of four elements
  const bool vec = d % 4 == 0 && dv % 4 == 0 && q_stride % 4 == 0 && k_stride % 4 == 0 && v_stride % 4 == 0 && qo_stride % 4 == 0 &&
                   (uintptr_t)q % ia == 0 && (uintptr_t)k % ia == 0 && (uintptr_t)v % ia == 0 && (uintptr_t)q_out % oa == 0 &&
                   (uintptr_t)k_cache % oa == 0 && (uintptr_t)v_cache % oa == 0;
#define QKN_GO(TI, TO, VEC) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(qk_norm_rope_write_kernel<TI, TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    return launch_pdl(qk_norm_rope_write_kernel<TI, TO, VEC>, grid, dim3(QKN_WARPS * 32), smem, stream, (const TI*)q, q_stride, \
        (const TI*)k, k_stride, (const TI*)v, v_stride, (TO*)q_out, qo_stride, q_w, k_w, wb, eps, positions, inv_freq, rot_dims, \
        slot_mapping, (TO*)k_cache, (TO*)v_cache, n_q, n_kv, d, dv, page_size, num_slots, err); } while (0)
#define QKN_LAUNCH(TI, TO) do { if (vec) QKN_GO(TI, TO, true); else QKN_GO(TI, TO, false); } while (0)
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) QKN_LAUNCH(float, float);
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) QKN_LAUNCH(float, bf16);
  if (in_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) QKN_LAUNCH(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}
