// Gated linear attention: a recurrent mixer whose state is one matrix per head, S [dim][vdim] in 32-bit.
// With a decay per key channel a_t = sigmoid(z_t)^(1/tau) (computed as exp(log_sigmoid(z_t) / tau)), whose
// logits are the second half of a low-rank projection, z_t = W_a2 low_t + b (low_t = W_a1 h_t comes in with
// q, k, v and g; the few multiply-adds per channel are done here, in 32-bit),
//
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T,        o_t = S_t^T (q_t * qscale),
//
// and the head's output is o_t divided by its root mean square over vdim (eps inside the root), times a
// weight shared by the heads, times silu(g_t).  One block owns one (request, head): it reads the state from
// the request's slot, walks the request's tokens of this step in order, and writes the state back, so a
// prompt portion, a single decoded token and a mixed batch are the same case, and a request's result does not
// depend on how it was cut into steps (the per-token arithmetic is the same chain either way).
//
// Thread r * vdim + j holds the state rows r * RPT .. r * RPT + RPT - 1 of value column j in registers; the partial
// sums over rows meet in shared memory in the order of r.  q, k and the decay of the next token are fetched
// while the current one is computed.  Everything is 32-bit; q, k, v and g may be stored as bfloat16.
#include "common.cuh"
#include <math.h>

template <typename T, int RPT>
__global__ void gla_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                     const T* __restrict__ g, const T* __restrict__ low, long in_stride, int rank,
                                     const T* __restrict__ w_a2, const void* __restrict__ b_a2, int b_bf16,
                                     const void* __restrict__ norm_w, int norm_w_bf16, float eps, float inv_tau,
                                     float qscale, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ state_slots, float* __restrict__ state, int num_slots,
                                     T* __restrict__ out, long out_stride, int heads, int dim, int vdim, int* err) {
  extern __shared__ float sm[];
  const int s = blockIdx.x, h = blockIdx.y;
  const int R = (dim + RPT - 1) / RPT;
  const int tid = threadIdx.x, nthreads = blockDim.x;                       // a whole number of warps
  const bool active = tid < vdim * R;                                        // the others only meet at barriers
  const int j = active ? tid % vdim : 0, r = active ? tid / vdim : R;
  float* qs = sm;                        // 2 x dim
  float* ks = qs + 2 * dim;              // 2 x dim
  float* as = ks + 2 * dim;              // 2 x dim
  float* part = as + 2 * dim;            // R x vdim
  float* red = part + R * vdim;          // 32
  float* wa = red + 32;                  // dim x (rank + 1): this head's rows of W_a2
  float* ba = wa + dim * (rank + 1);     // dim
  const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
  if (t1 <= t0) return;
  const int slot = state_slots[s];
  if (slot >= num_slots) {
    if (tid == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t0, slot, num_slots);
    return;
  }
  float* S = slot >= 0 ? state + ((size_t)slot * heads + h) * dim * vdim : nullptr;
  float st[RPT];
  const int row0 = r * RPT;
#pragma unroll
  for (int i = 0; i < RPT; ++i) st[i] = (S != nullptr && active && row0 + i < dim) ? S[(size_t)(row0 + i) * vdim + j] : 0.f;
  const float wj = load_w(norm_w, norm_w_bf16, j);
  for (int i = tid; i < dim * rank; i += nthreads) wa[(i / rank) * (rank + 1) + i % rank] = to_f32(w_a2[(size_t)h * dim * rank + i]);
  for (int i = tid; i < dim; i += nthreads) ba[i] = load_w(b_a2, b_bf16, (size_t)h * dim + i);
  __syncthreads();

  auto fetch = [&](int t, int buf) {
    for (int i = tid; i < dim; i += nthreads) {
      const size_t off = (size_t)t * in_stride + (size_t)h * dim + i;
      qs[buf * dim + i] = to_f32(q[off]) * qscale;
      ks[buf * dim + i] = to_f32(k[off]);
      const T* lw = low + (size_t)t * in_stride;
      float zz = 0.f;
      for (int c = 0; c < rank; ++c) zz = fmaf(to_f32(lw[c]), wa[i * (rank + 1) + c], zz);
      zz += ba[i];
      const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));          // log(sigmoid(z))
      as[buf * dim + i] = expf(ls * inv_tau);
    }
  };
  fetch(t0, 0);
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    if (t + 1 < t1) fetch(t + 1, buf ^ 1);
    const float vj = to_f32(v[(size_t)t * in_stride + (size_t)h * vdim + j]);
    const float* qb = qs + buf * dim + row0;
    const float* kb = ks + buf * dim + row0;
    const float* ab = as + buf * dim + row0;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      if (row0 + i < dim) {
        st[i] = fmaf(ab[i], st[i], kb[i] * vj);
        o = fmaf(st[i], qb[i], o);
      }
    }
    if (active) part[r * vdim + j] = o;
    __syncthreads();
    float tot = 0.f, sq = 0.f;
    if (r == 0) {
      for (int rr = 0; rr < R; ++rr) tot += part[rr * vdim + j];
      sq = tot * tot;
    }
    sq = block_sum(sq, red);                               // two barriers inside: `part` and the next token's
    if (r == 0) {                                          // q, k and decay are settled when it returns
      const float inv = 1.0f / sqrtf(sq / (float)vdim + eps);
      const float gg = to_f32(g[(size_t)t * in_stride + (size_t)h * vdim + j]);
      out[(size_t)t * out_stride + (size_t)h * vdim + j] = from_f32<T>(tot * inv * wj * (gg / (1.0f + expf(-gg))));
    }
  }
  if (S != nullptr && active) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (row0 + i < dim) S[(size_t)(row0 + i) * vdim + j] = st[i];
  }
}

template <typename T, int RPT>
static int gla_launch(const void* q, const void* k, const void* v, const void* g, const void* low, long in_stride,
                      int rank, const void* w_a2, const void* b_a2, int b_bf16, const void* norm_w, int norm_w_bf16, float eps, float inv_tau, float qscale,
                      const int* cu_tokens, const int* state_slots, float* state, int num_slots, void* out,
                      long out_stride, int S, int heads, int dim, int vdim, int* err, cudaStream_t stream) {
  const int R = (dim + RPT - 1) / RPT;
  if (vdim * R > 1024) return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)7 * dim + (size_t)R * vdim + 32 + (size_t)dim * (rank + 1)) * sizeof(float);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gla_recurrent_kernel<T, RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  gla_recurrent_kernel<T, RPT><<<dim3(S, heads), dim3((vdim * R + 31) / 32 * 32), smem, stream>>>(
      (const T*)q, (const T*)k, (const T*)v, (const T*)g, (const T*)low, in_stride, rank, (const T*)w_a2, b_a2, b_bf16,
      norm_w, norm_w_bf16, eps, inv_tau,
      qscale, cu_tokens, state_slots, state, num_slots, (T*)out, out_stride, heads, dim, vdim, err);
  return launch_status();
}

// q, k [T][heads * dim], v, g [T][heads * vdim], low [T][rank]: sections of one fused row (one row stride, in
// elements).  w_a2 [heads * dim][rank] (the type of q), b_a2 [heads * dim]: the decay logits are w_a2 low + b_a2.  state [num_slots][heads][dim][vdim] float; a request whose slot
// is negative starts from zero and stores nothing.  out [T][heads * vdim].
PHOTON_API int photon_gla_recurrent(const void* q, const void* k, const void* v, const void* g, const void* low,
                                    long in_stride, int dtype, int rank, const void* w_a2, const void* b_a2,
                                    int b_a2_dtype, const void* norm_w, int norm_w_dtype,
                                    float eps, float tau, float qscale, const int* cu_tokens, const int* state_slots,
                                    float* state, int num_slots, void* out, long out_stride, int S, int heads, int dim,
                                    int vdim, int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || rank <= 0 || !(tau > 0.f)) return PHOTON_ERR_ARGUMENT;
  const int bb = b_a2_dtype == PHOTON_BF16;
  if (heads > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int wb = norm_w_dtype == PHOTON_BF16;
  const float it = 1.0f / tau;
  // rows of the state per thread: as few as keep the block within 1024 threads
  int rpt = 8;
  while (rpt < 64 && (long)vdim * ((dim + rpt - 1) / rpt) > 512) rpt *= 2;
#define GLA_ARGS q, k, v, g, low, in_stride, rank, w_a2, b_a2, bb, norm_w, wb, eps, it, qscale, cu_tokens, state_slots, state, \
                 num_slots, out, out_stride, S, heads, dim, vdim, err, stream
  if (dtype == PHOTON_BF16) {
    if (rpt == 8) return gla_launch<bf16, 8>(GLA_ARGS);
    if (rpt == 16) return gla_launch<bf16, 16>(GLA_ARGS);
    if (rpt == 32) return gla_launch<bf16, 32>(GLA_ARGS);
    return gla_launch<bf16, 64>(GLA_ARGS);
  }
  if (rpt == 8) return gla_launch<float, 8>(GLA_ARGS);
  if (rpt == 16) return gla_launch<float, 16>(GLA_ARGS);
  if (rpt == 32) return gla_launch<float, 32>(GLA_ARGS);
  return gla_launch<float, 64>(GLA_ARGS);
}
