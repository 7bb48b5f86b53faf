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

template <typename TI, typename TO>
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
      for (int i = lane; i < dv; i += 32) dst[i] = from_f32<TO>(to_f32(vr[i]));
    }
    return;
  }
  const TI* row = (which == 0 ? q + (size_t)t * q_stride : k + (size_t)t * k_stride) + (size_t)h * d;
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) { const float x = to_f32(row[i]); xs[i] = x; ss += x * x; }
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
  if (which == 0) {
    TO* dst = q_out + (size_t)t * qo_stride + (size_t)h * d;
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<TO>(xs[i]);
  } else if (slot >= 0) {
    TO* dst = k_cache + page_at * d;
    for (int i = lane; i < d; i += 32) dst[i] = from_f32<TO>(xs[i]);
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
#define QKN_LAUNCH(TI, TO) do { \
    if (smem > 48 * 1024) { cudaError_t e_ = cudaFuncSetAttribute(qk_norm_rope_write_kernel<TI, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
                            if (e_ != cudaSuccess) return (int)e_; } \
    return launch_pdl(qk_norm_rope_write_kernel<TI, TO>, grid, dim3(QKN_WARPS * 32), smem, stream, (const TI*)q, q_stride, \
        (const TI*)k, k_stride, (const TI*)v, v_stride, (TO*)q_out, qo_stride, q_w, k_w, wb, eps, positions, inv_freq, rot_dims, \
        slot_mapping, (TO*)k_cache, (TO*)v_cache, n_q, n_kv, d, dv, page_size, num_slots, err); } while (0)
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_F32) QKN_LAUNCH(float, float);
  if (in_dtype == PHOTON_F32 && out_dtype == PHOTON_BF16) QKN_LAUNCH(float, bf16);
  if (in_dtype == PHOTON_BF16 && out_dtype == PHOTON_BF16) QKN_LAUNCH(bf16, bf16);
  return PHOTON_ERR_ARGUMENT;
}
