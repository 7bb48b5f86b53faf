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

// Rows of the state per thread and the block's width: as few rows as keep the block within 256 threads (then a
// thread may use 255 registers and nothing spills), else within 512.
static inline void gla_shape(int dim, int vdim, int* rpt, int* maxt) {
  // the narrowest block that holds the state with at most 64 rows a thread: 256 threads may use 255 registers each
  // and nothing spills.  Measured at heads of 128 x 128: blocks of 256, 512 and 1024 threads take the same time.
  for (int limit = 256; limit <= 1024; limit *= 2) {
    for (int r = 8; r <= 64; r *= 2) {
      if ((long)vdim * ((dim + r - 1) / r) <= limit && dim <= limit) { *rpt = r; *maxt = limit; return; }
    }
  }
  *rpt = 64; *maxt = 1024;                               // refused by the launcher when it does not fit
}

// skip_from > 0: requests that bring that many tokens or more are left to the chunked kernels below.
template <typename T, int RPT, int MAXT>
__global__ void __launch_bounds__(MAXT) gla_recurrent_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                                     const T* __restrict__ g, const T* __restrict__ low, long in_stride, int rank,
                                     const T* __restrict__ w_a2, const void* __restrict__ b_a2, int b_bf16,
                                     const void* __restrict__ norm_w, int norm_w_bf16, float eps, float inv_tau,
                                     float qscale, const int* __restrict__ cu_tokens,
                                     const int* __restrict__ state_slots, float* __restrict__ state, int num_slots,
                                     T* __restrict__ out, long out_stride, int heads, int dim, int vdim, int* err,
                                     int skip_from) {
  extern __shared__ float sm[];
  const int s = blockIdx.x, h = blockIdx.y;
  const int R = (dim + RPT - 1) / RPT;
  const int tid = threadIdx.x, nthreads = blockDim.x;                       // a whole number of warps
  const bool active = tid < vdim * R;                                        // the others only meet at barriers
  const int j = active ? tid % vdim : 0, r = active ? tid / vdim : R;
  const int dimp = R * RPT;              // rows padded to whole groups: the padding stays zero and adds nothing
  float* qs = sm;                        // 2 x dimp
  float* ks = qs + 2 * dimp;             // 2 x dimp
  float* as = ks + 2 * dimp;             // 2 x dimp
  float* part = as + 2 * dimp;           // R x vdim
  float* red = part + R * vdim;          // 32
  float* wa = red + 32;                  // dim x (rank + 1): this head's rows of W_a2
  float* ba = wa + dim * (rank + 1);     // dim
  const int t0 = cu_tokens[s], t1 = cu_tokens[s + 1];
  if (t1 <= t0 || (skip_from > 0 && t1 - t0 >= skip_from)) return;        // long portions go the chunked way
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
  for (int i = tid; i < 6 * dimp; i += nthreads) sm[i] = 0.f;
  for (int i = tid; i < dim * rank; i += nthreads) wa[(i / rank) * (rank + 1) + i % rank] = to_f32(w_a2[(size_t)h * dim * rank + i]);
  for (int i = tid; i < dim; i += nthreads) ba[i] = load_w(b_a2, b_bf16, (size_t)h * dim + i);
  __syncthreads();

  // Two tokens ahead: the raw q, k and low-rank row of token t + 1 wait in registers while token t is computed, and
  // become the decayed inputs in shared memory right before they are needed; v and g of the next token likewise.
  // A block has at least `dim` threads, so thread i < dim owns decay channel i.
  constexpr int LR = MAXT >= 1024 ? 8 : 16;              // low-rank values kept in registers; more are read late
  const bool owner = tid < dim;
  float rq = 0.f, rk = 0.f, rl[LR];
  auto load = [&](int t) {
    if (!owner) return;
    const size_t off = (size_t)t * in_stride + (size_t)h * dim + tid;
    rq = to_f32(q[off]);
    rk = to_f32(k[off]);
    const T* lw = low + (size_t)t * in_stride;
#pragma unroll
    for (int c = 0; c < LR; ++c) rl[c] = c < rank ? to_f32(lw[c]) : 0.f;
  };
  auto commit = [&](int t, int buf) {
    if (!owner) return;
    const int i = tid;
    float zz = 0.f;
#pragma unroll
    for (int c = 0; c < LR; ++c) if (c < rank) zz = fmaf(rl[c], wa[i * (rank + 1) + c], zz);
    const T* lw = low + (size_t)t * in_stride;
    for (int c = LR; c < rank; ++c) zz = fmaf(to_f32(lw[c]), wa[i * (rank + 1) + c], zz);
    zz += ba[i];
    const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));            // log(sigmoid(z))
    const float a = expf(ls * inv_tau);
    qs[buf * dimp + i] = rq * qscale;
    ks[buf * dimp + i] = rk;
    as[buf * dimp + i] = a;
  };
  load(t0);
  commit(t0, 0);
  if (t0 + 1 < t1) load(t0 + 1);
  float vj = to_f32(v[(size_t)t0 * in_stride + (size_t)h * vdim + j]);
  float gj = to_f32(g[(size_t)t0 * in_stride + (size_t)h * vdim + j]);
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const int buf = (t - t0) & 1;
    if (t + 1 < t1) commit(t + 1, buf ^ 1);              // its raw values arrived during the last token
    if (t + 2 < t1) load(t + 2);
    const float vcur = vj, gcur = gj;
    if (t + 1 < t1) {
      vj = to_f32(v[(size_t)(t + 1) * in_stride + (size_t)h * vdim + j]);
      gj = to_f32(g[(size_t)(t + 1) * in_stride + (size_t)h * vdim + j]);
    }
    float o = 0.f;
    if (active) {
      // a thread's rows lie side by side: four decays, keys and queries per shared-memory read
      const float4* qb = reinterpret_cast<const float4*>(qs + buf * dimp + row0);
      const float4* kb = reinterpret_cast<const float4*>(ks + buf * dimp + row0);
      const float4* ab = reinterpret_cast<const float4*>(as + buf * dimp + row0);
      float o2 = 0.f;
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 a4 = ab[i], k4 = kb[i], q4 = qb[i];
        st[4 * i] = fmaf(a4.x, st[4 * i], k4.x * vcur);
        st[4 * i + 1] = fmaf(a4.y, st[4 * i + 1], k4.y * vcur);
        st[4 * i + 2] = fmaf(a4.z, st[4 * i + 2], k4.z * vcur);
        st[4 * i + 3] = fmaf(a4.w, st[4 * i + 3], k4.w * vcur);
        o = fmaf(st[4 * i], q4.x, o);
        o2 = fmaf(st[4 * i + 1], q4.y, o2);
        o = fmaf(st[4 * i + 2], q4.z, o);
        o2 = fmaf(st[4 * i + 3], q4.w, o2);
      }
      o += o2;
      part[r * vdim + j] = o;
    }
    __syncthreads();
    float tot = 0.f, sq = 0.f;
    if (r == 0) {
      for (int rr = 0; rr < R; ++rr) tot += part[rr * vdim + j];
      sq = tot * tot;
    }
    sq = block_sum(sq, red);                               // two barriers inside: `part` and the next token's
    if (r == 0) {                                          // q, k and decay are settled when it returns
      const float inv = 1.0f / sqrtf(sq / (float)vdim + eps);
      out[(size_t)t * out_stride + (size_t)h * vdim + j] = from_f32<T>(tot * inv * wj * (gcur / (1.0f + expf(-gcur))));
    }
  }
  if (S != nullptr && active) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (row0 + i < dim) S[(size_t)(row0 + i) * vdim + j] = st[i];
  }
}

// ---------------------------------------------------------------- one chunk of a long portion, from a zero state
// Everything the chunk needs is brought into shared memory at once (decayed inputs of all its tokens, formed side
// by side), the walk over its tokens then touches no global memory but its results and meets no barrier: thread
// j * RP + r keeps rows r * RPT .. of column j, and the RP partial sums of a column lie in neighbouring lanes and
// meet by shuffles.  Leaves the chunk's own outputs o_loc [T][heads][vdim] (no norm yet), the decay from the chunk's
// start through every token b [T][heads][dim], and the chunk's end state s_loc [chunks][heads][dim][vdim].
template <typename T, int RPT>
__global__ void __launch_bounds__(512)
gla_chunk_local_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                       const T* __restrict__ low, long in_stride, int rank, const T* __restrict__ w_a2,
                       const void* __restrict__ b_a2, int b_bf16, float inv_tau, float qscale, int first, int count,
                       int chunk, float* __restrict__ o_loc, float* __restrict__ b_out, float* __restrict__ s_loc,
                       int heads, int dim, int vdim, int RP) {
  extern __shared__ __align__(16) float sm[];
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, nthreads = blockDim.x;
  const int R = (dim + RPT - 1) / RPT;
  const int gs = RPT + 4;                  // a row group's stride: groups start in different banks
  const int dimp = R * gs;
  const int t0 = first + c * chunk, n = min(first + count, t0 + chunk) - t0;
  float* qf = sm;                          // chunk x dimp
  float* kf = qf + chunk * dimp;
  float* af = kf + chunk * dimp;
  float* vf = af + chunk * dimp;           // chunk x vdim
  float* wa = vf + chunk * vdim;           // dim x (rank + 1)
  float* ba = wa + dim * (rank + 1);       // dim
  for (int i = tid; i < dim * rank; i += nthreads) wa[(i / rank) * (rank + 1) + i % rank] = to_f32(w_a2[(size_t)h * dim * rank + i]);
  for (int i = tid; i < dim; i += nthreads) ba[i] = load_w(b_a2, b_bf16, (size_t)h * dim + i);
  for (int i = tid; i < 3 * chunk * dimp; i += nthreads) sm[i] = 0.f;
  __syncthreads();
  for (int e = tid; e < n * dim; e += nthreads) {
    const int t = e / dim, i = e - t * dim;
    const size_t off = (size_t)(t0 + t) * in_stride + (size_t)h * dim + i;
    const T* lw = low + (size_t)(t0 + t) * in_stride;
    float zz = 0.f;
    for (int r = 0; r < rank; ++r) zz = fmaf(to_f32(lw[r]), wa[i * (rank + 1) + r], zz);
    zz += ba[i];
    const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));            // log(sigmoid(z))
    const int at = t * dimp + (i / RPT) * gs + i % RPT;
    qf[at] = to_f32(q[off]) * qscale;
    kf[at] = to_f32(k[off]);
    af[at] = expf(ls * inv_tau);
  }
  for (int e = tid; e < n * vdim; e += nthreads) {
    const int t = e / vdim, j = e - t * vdim;
    vf[e] = to_f32(v[(size_t)(t0 + t) * in_stride + (size_t)h * vdim + j]);
  }
  __syncthreads();
  if (tid < dim) {                          // the decay since the chunk's start, channel by channel
    float cum = 1.f;
    const int at = (tid / RPT) * gs + tid % RPT;
    for (int t = 0; t < n; ++t) {
      cum *= af[t * dimp + at];
      b_out[((size_t)(t0 + t) * heads + h) * dim + tid] = cum;
    }
  }
  const int j = tid / RP, r = tid % RP;
  const bool active = j < vdim && r < R;
  float st[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) st[i] = 0.f;
  const int g0 = (r < R ? r : 0) * gs;
  for (int t = 0; t < n; ++t) {
    float o = 0.f, o2 = 0.f;
    if (active) {
      const float vcur = vf[t * vdim + j];
      const float4* qb = reinterpret_cast<const float4*>(qf + t * dimp + g0);
      const float4* kb = reinterpret_cast<const float4*>(kf + t * dimp + g0);
      const float4* ab = reinterpret_cast<const float4*>(af + t * dimp + g0);
#pragma unroll
      for (int i = 0; i < RPT / 4; ++i) {
        const float4 a4 = ab[i], k4 = kb[i], q4 = qb[i];
        st[4 * i] = fmaf(a4.x, st[4 * i], k4.x * vcur);
        st[4 * i + 1] = fmaf(a4.y, st[4 * i + 1], k4.y * vcur);
        st[4 * i + 2] = fmaf(a4.z, st[4 * i + 2], k4.z * vcur);
        st[4 * i + 3] = fmaf(a4.w, st[4 * i + 3], k4.w * vcur);
        o = fmaf(st[4 * i], q4.x, o);
        o2 = fmaf(st[4 * i + 1], q4.y, o2);
        o = fmaf(st[4 * i + 2], q4.z, o);
        o2 = fmaf(st[4 * i + 3], q4.w, o2);
      }
      o += o2;
    }
    for (int d = 1; d < RP; d <<= 1) o += __shfl_xor_sync(0xffffffffu, o, d);   // RP lanes of a column, fixed order
    if (active && r == 0) o_loc[((size_t)(t0 + t) * heads + h) * vdim + j] = o;
  }
  if (active) {
    float* S = s_loc + ((size_t)c * heads + h) * dim * vdim;
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (r * RPT + i < dim) S[(size_t)(r * RPT + i) * vdim + j] = st[i];
  }
}

template <typename T, int RPT>
static int gla_chunk_local_launch(const void* q, const void* k, const void* v, const void* low, long in_stride, int rank,
                                  const void* w_a2, const void* b_a2, int bb, float it, float qscale, int first, int count,
                                  int chunk, float* o_loc, float* b, float* s_loc, int heads, int dim, int vdim, int rp,
                                  int chunks, cudaStream_t stream) {
  const int R = (dim + RPT - 1) / RPT;
  const size_t smem = ((size_t)3 * chunk * R * (RPT + 4) + (size_t)chunk * vdim + (size_t)dim * (rank + 2)) * sizeof(float);
  int threads = (vdim * rp + 31) / 32 * 32;
  if (threads < dim) threads = (dim + 31) / 32 * 32;
  if (threads > 512 || smem > 220 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gla_chunk_local_kernel<T, RPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  gla_chunk_local_kernel<T, RPT><<<dim3(chunks, heads), threads, smem, stream>>>(
      (const T*)q, (const T*)k, (const T*)v, (const T*)low, in_stride, rank, (const T*)w_a2, b_a2, bb, it, qscale, first,
      count, chunk, o_loc, b, s_loc, heads, dim, vdim, rp);
  return launch_status();
}

// Rows per thread of the chunk kernel: the fewest with which the block (columns x row groups, the groups rounded up to a
// power of two so that they meet by shuffles) stays within 512 threads.  0: no shape fits.
static inline int gla_chunk_rows(int dim, int vdim, int* rp) {
  for (int r = 8; r <= 64; r *= 2) {
    const int R = (dim + r - 1) / r;
    int p = 1;
    while (p < R) p <<= 1;
    if (p <= 32 && (long)vdim * p <= 512 && dim <= 512) { *rp = p; return r; }
  }
  return 0;
}

// The states at the chunks' starts, one (i, j) element per thread, chunk after chunk: start[0] is the state in the
// request's slot (zero for a negative slot), start[c + 1] = b_end[c] * start[c] + s_loc[c]; s_loc[c] is overwritten
// with start[c], and the state after the last chunk goes back into the slot.
__global__ void gla_chunk_scan_kernel(float* s_loc, const float* __restrict__ b, int first, int count,
                                      int chunk, int chunks, float* __restrict__ state, int slot, int heads, int dim,
                                      int vdim) {
  const int h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= dim * vdim) return;
  const int i = e / vdim;
  float* S = slot >= 0 ? state + ((size_t)slot * heads + h) * dim * vdim : nullptr;
  float cur = S ? S[e] : 0.f;
  auto decay_of = [&](int c) { return b[((size_t)(min(first + count, first + (c + 1) * chunk) - 1) * heads + h) * dim + i]; };
  auto end_of = [&](int c) { return s_loc[((size_t)c * heads + h) * dim * vdim + e]; };
  // four chunks' values are on their way before the first of them is used
  constexpr int AHEAD = 4;
  float bd[AHEAD], le[AHEAD];
#pragma unroll
  for (int u = 0; u < AHEAD; ++u) { bd[u] = u < chunks ? decay_of(u) : 0.f; le[u] = u < chunks ? end_of(u) : 0.f; }
  for (int c0 = 0; c0 < chunks; c0 += AHEAD) {
    float nb[AHEAD], nl[AHEAD];
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int c = c0 + AHEAD + u;
      nb[u] = c < chunks ? decay_of(c) : 0.f;
      nl[u] = c < chunks ? end_of(c) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) {
      const int c = c0 + u;
      if (c < chunks) {
        s_loc[((size_t)c * heads + h) * dim * vdim + e] = cur;
        cur = fmaf(bd[u], cur, le[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < AHEAD; ++u) { bd[u] = nb[u]; le[u] = nl[u]; }
  }
  if (S) S[e] = cur;
}

// What the state at the chunk's start adds to every token of the chunk, o_t += sum_i (q_t[i] b_t[i]) start[i][:],
// then the head's norm and the gate.  One block per (chunk, head); the start state and the decayed queries in shared
// memory.
template <typename T>
__global__ void __launch_bounds__(256)
gla_chunk_out_kernel(const T* __restrict__ q, const T* __restrict__ g, long in_stride, const float* __restrict__ b,
                     const float* __restrict__ o_loc, const float* __restrict__ s_start, const void* __restrict__ norm_w,
                     int norm_w_bf16, float eps, float qscale, int first, int count, int chunk, T* __restrict__ out,
                     long out_stride, int heads, int dim, int vdim) {
  extern __shared__ float sm[];
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int t0 = first + c * chunk, n = min(first + count, t0 + chunk) - t0;
  float* Ss = sm;                         // dim x vdim
  const int qld = chunk + 4;                  // a channel's stride in qb: neighbouring channels start four banks apart
  float* qb = Ss + ((dim * vdim + 3) & ~3);   // dim x qld, 16-byte aligned
  float* os = qb + qld * dim;             // chunk x vdim
  const float* src = s_start + ((size_t)c * heads + h) * dim * vdim;
  if ((dim * vdim) % 4 == 0) {
    for (int e = tid; e < dim * vdim / 4; e += 256) reinterpret_cast<float4*>(Ss)[e] = reinterpret_cast<const float4*>(src)[e];
  } else {
    for (int e = tid; e < dim * vdim; e += 256) Ss[e] = src[e];
  }
  // the decayed queries, transposed: qb[i][t], so that eight tokens of one channel are two 16-byte reads
  for (int e = tid; e < chunk * dim; e += 256) {
    const int t = e / dim, i = e - t * dim;
    qb[i * qld + t] = t < n ? to_f32(q[(size_t)(t0 + t) * in_stride + (size_t)h * dim + i]) * qscale *
                                    b[((size_t)(t0 + t) * heads + h) * dim + i] : 0.f;
  }
  __syncthreads();
  // a thread owns four value columns and eight tokens: three 16-byte reads of shared memory serve 32 multiply-adds
  const int groups = chunk / 8, quads = (vdim + 3) / 4;
  const bool vec4 = (vdim & 3) == 0;
  for (int e = tid; e < groups * quads; e += 256) {
    const int tg = e / quads, j = (e - tg * quads) * 4;
    float a[8][4];
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int w = 0; w < 4; ++w) a[u][w] = 0.f;
    for (int i = 0; i < dim; ++i) {
      float sv[4];
      if (vec4) {
        const float4 s4 = *reinterpret_cast<const float4*>(Ss + i * vdim + j);
        sv[0] = s4.x; sv[1] = s4.y; sv[2] = s4.z; sv[3] = s4.w;
      } else {
#pragma unroll
        for (int w = 0; w < 4; ++w) sv[w] = j + w < vdim ? Ss[i * vdim + j + w] : 0.f;
      }
      const float4 q0 = *reinterpret_cast<const float4*>(qb + i * qld + tg * 8);
      const float4 q1 = *reinterpret_cast<const float4*>(qb + i * qld + tg * 8 + 4);
      const float qv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int w = 0; w < 4; ++w) a[u][w] = fmaf(qv[u], sv[w], a[u][w]);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int t = tg * 8 + u;
      if (t < n) {
#pragma unroll
        for (int w = 0; w < 4; ++w)
          if (j + w < vdim) os[t * vdim + j + w] = a[u][w] + o_loc[((size_t)(t0 + t) * heads + h) * vdim + j + w];
      }
    }
  }
  __syncthreads();
  const int warp = tid >> 5, lane = tid & 31;
  for (int t = warp; t < n; t += 8) {
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss += os[t * vdim + j] * os[t * vdim + j];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)vdim + eps);
    for (int j = lane; j < vdim; j += 32) {
      const float gg = to_f32(g[(size_t)(t0 + t) * in_stride + (size_t)h * vdim + j]);
      out[(size_t)(t0 + t) * out_stride + (size_t)h * vdim + j] =
          from_f32<T>(os[t * vdim + j] * inv * load_w(norm_w, norm_w_bf16, j) * (gg / (1.0f + expf(-gg))));
    }
  }
}

template <typename T, int RPT, int MAXT>
static int gla_launch(const void* q, const void* k, const void* v, const void* g, const void* low, long in_stride,
                      int rank, const void* w_a2, const void* b_a2, int b_bf16, const void* norm_w, int norm_w_bf16, float eps, float inv_tau, float qscale,
                      const int* cu_tokens, const int* state_slots, float* state, int num_slots, void* out,
                      long out_stride, int S, int heads, int dim, int vdim, int* err, cudaStream_t stream, int skip_from) {
  const int R = (dim + RPT - 1) / RPT;
  if (vdim * R > MAXT) return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = ((size_t)6 * R * RPT + dim + (size_t)R * vdim + 32 + (size_t)dim * (rank + 1)) * sizeof(float);
  if (smem > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(gla_recurrent_kernel<T, RPT, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  int threads = (vdim * R + 31) / 32 * 32;
  if (threads < dim) threads = (dim + 31) / 32 * 32;                  // thread i < dim owns decay channel i
  if (threads > MAXT) return PHOTON_ERR_UNSUPPORTED;
  gla_recurrent_kernel<T, RPT, MAXT><<<dim3(S, heads), dim3(threads), smem, stream>>>(
      (const T*)q, (const T*)k, (const T*)v, (const T*)g, (const T*)low, in_stride, rank, (const T*)w_a2, b_a2, b_bf16,
      norm_w, norm_w_bf16, eps, inv_tau,
      qscale, cu_tokens, state_slots, state, num_slots, (T*)out, out_stride, heads, dim, vdim, err, skip_from);
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
                                    int vdim, int skip_from, int* err, cudaStream_t stream) {
  if (S <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || rank <= 0 || !(tau > 0.f)) return PHOTON_ERR_ARGUMENT;
  const int bb = b_a2_dtype == PHOTON_BF16;
  if (heads > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int wb = norm_w_dtype == PHOTON_BF16;
  const float it = 1.0f / tau;
  int rpt = 0, maxt = 256;
  gla_shape(dim, vdim, &rpt, &maxt);
#define GLA_ARGS q, k, v, g, low, in_stride, rank, w_a2, b_a2, bb, norm_w, wb, eps, it, qscale, cu_tokens, state_slots, state, \
                 num_slots, out, out_stride, S, heads, dim, vdim, err, stream
#define GLA_DISPATCH_T(MAXT)                                                      \
  if (dtype == PHOTON_BF16) {                                                     \
    if (rpt == 8) return gla_launch<bf16, 8, MAXT>(GLA_ARGS, skip_from);          \
    if (rpt == 16) return gla_launch<bf16, 16, MAXT>(GLA_ARGS, skip_from);        \
    if (rpt == 32) return gla_launch<bf16, 32, MAXT>(GLA_ARGS, skip_from);        \
    return gla_launch<bf16, 64, MAXT>(GLA_ARGS, skip_from);                       \
  }                                                                               \
  if (rpt == 8) return gla_launch<float, 8, MAXT>(GLA_ARGS, skip_from);           \
  if (rpt == 16) return gla_launch<float, 16, MAXT>(GLA_ARGS, skip_from);         \
  if (rpt == 32) return gla_launch<float, 32, MAXT>(GLA_ARGS, skip_from);         \
  return gla_launch<float, 64, MAXT>(GLA_ARGS, skip_from);
  if (maxt == 1024) { GLA_DISPATCH_T(1024) }
  if (maxt == 512) { GLA_DISPATCH_T(512) }
  GLA_DISPATCH_T(256)
}

// One long prompt portion (tokens first .. first + count - 1 of the step, state slot `slot`) in chunks that run side by
// side: every chunk's own recurrence from zero, a scan over the chunks' end states, and the start states' share of the
// outputs with the norm and the gate.  scratch: float [count * heads * (vdim + dim) + 4 + chunks * heads * dim * vdim]
// with chunks = ceil(count / chunk), 16-byte aligned.  The sums differ from the token-by-token kernel's in their order only.
PHOTON_API int photon_gla_chunked(const void* q, const void* k, const void* v, const void* g, const void* low,
                                  long in_stride, int dtype, int rank, const void* w_a2, const void* b_a2, int b_a2_dtype,
                                  const void* norm_w, int norm_w_dtype, float eps, float tau, float qscale, int first,
                                  int count, int chunk, int slot, float* state, int num_slots, float* scratch, void* out,
                                  long out_stride, int heads, int dim, int vdim, int* err, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (heads <= 0 || dim <= 0 || vdim <= 0 || rank <= 0 || chunk <= 0 || chunk % 8 || !(tau > 0.f) || slot >= num_slots)
    return PHOTON_ERR_ARGUMENT;
  if (heads > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int chunks = (count + chunk - 1) / chunk;
  const size_t smem_out = ((size_t)dim * vdim + 4 + (size_t)(chunk + 4) * dim + (size_t)chunk * vdim) * sizeof(float);
  if (smem_out > 200 * 1024) return PHOTON_ERR_UNSUPPORTED;
  // the scratch is indexed by the token's place in the step: its three parts are laid out for tokens first ..
  float* o_loc = scratch - (size_t)first * heads * vdim;
  float* b = scratch + (size_t)count * heads * vdim - (size_t)first * heads * dim;
  float* s_loc = scratch + (((size_t)count * heads * (vdim + dim) + 3) & ~(size_t)3);   // 16-byte aligned: read four at a time
  const int wb = norm_w_dtype == PHOTON_BF16, bb = b_a2_dtype == PHOTON_BF16;
  const float it = 1.0f / tau;
  int rp = 1;
  const int rows = gla_chunk_rows(dim, vdim, &rp);
  if (rows == 0) return PHOTON_ERR_UNSUPPORTED;
  int st;
#define GLA_LOCAL(T, RPT) gla_chunk_local_launch<T, RPT>(q, k, v, low, in_stride, rank, w_a2, b_a2, bb, it, qscale, first, \
                                                         count, chunk, o_loc, b, s_loc, heads, dim, vdim, rp, chunks, stream)
  if (dtype == PHOTON_BF16) st = rows == 8 ? GLA_LOCAL(bf16, 8) : rows == 16 ? GLA_LOCAL(bf16, 16) : rows == 32 ? GLA_LOCAL(bf16, 32) : GLA_LOCAL(bf16, 64);
  else st = rows == 8 ? GLA_LOCAL(float, 8) : rows == 16 ? GLA_LOCAL(float, 16) : rows == 32 ? GLA_LOCAL(float, 32) : GLA_LOCAL(float, 64);
  if (st != 0) return st;
  gla_chunk_scan_kernel<<<dim3((dim * vdim + 255) / 256, heads), 256, 0, stream>>>(s_loc, b, first, count, chunk, chunks,
                                                                                state, slot, heads, dim, vdim);
  if ((st = launch_status()) != 0) return st;
  if (dtype == PHOTON_BF16) {
    if (smem_out > 48 * 1024) cudaFuncSetAttribute(gla_chunk_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
    gla_chunk_out_kernel<bf16><<<dim3(chunks, heads), 256, smem_out, stream>>>((const bf16*)q, (const bf16*)g, in_stride, b, o_loc,
        s_loc, norm_w, wb, eps, qscale, first, count, chunk, (bf16*)out, out_stride, heads, dim, vdim);
  } else {
    if (smem_out > 48 * 1024) cudaFuncSetAttribute(gla_chunk_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_out);
    gla_chunk_out_kernel<float><<<dim3(chunks, heads), 256, smem_out, stream>>>((const float*)q, (const float*)g, in_stride, b, o_loc,
        s_loc, norm_w, wb, eps, qscale, first, count, chunk, (float*)out, out_stride, heads, dim, vdim);
  }
  return launch_status();
}
