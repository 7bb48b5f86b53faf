// Kernels of attention over a cached latent: every token stores ONE row [c ; k_r] of kv_rank + rot numbers,
// the normed latent c and a rotated key part k_r shared by all heads.  A head's unrotated key is W_uk c and
// its value W_uv c; neither is ever formed.  With q_abs = W_uk^T q_unrotated the score of a head is
// (q_abs . c + q_r . k_r) * scale, the weighted sum of the latents is taken per head, and W_uv is applied to
// that sum.  The attention itself is photon_paged_attention with one key/value head whose values are the head
// of the key rows; this file holds what comes before and after it:
//
//   photon_latent_prep      one pass over the fused down-projection row of a token: RMS norm of the query
//                           latent, RMS norm of the key/value latent, rotation of the shared key part, and the
//                           row's write into the paged cache;
//   photon_latent_q_rope    the rotated part of every head's query, copied behind the absorbed part;
//   photon_head_linear      out[t, h, :] = W[h] x[t, h, :] for all heads in one launch (the absorption of W_uk
//                           into the queries and the application of W_uv to the attention result).
//
// Rotation: the first rot_dims numbers of the rotated part, feature i paired with i + rot_dims / 2, angle
// position * inv_freq[i] in 32-bit; features beyond rot_dims pass unchanged.  All arithmetic is 32-bit.
#include "common.cuh"
#include <math.h>

// ---------------------------------------------------------------- norms, rotation, cache write
template <typename T>
__global__ void latent_prep_kernel(const T* __restrict__ down, long down_stride, int q_rank, int kv_rank, int rot,
                                   int rot_dims, const void* __restrict__ qw, int qw_bf16,
                                   const void* __restrict__ kw, int kw_bf16, float eps,
                                   const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                   const int* __restrict__ slot_mapping, T* __restrict__ cq, long cq_stride,
                                   T* __restrict__ cache, long num_slots, int* err) {
  __shared__ float red[32];
  const int t = blockIdx.x;
  const T* row = down + (size_t)t * down_stride;
  // query latent
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_f32(row[i]); ss += v * v; }
  ss = block_sum(ss, red);
  const float qinv = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * cq_stride + i] = from_f32<T>(to_f32(row[i]) * qinv * load_w(qw, qw_bf16, i));
  // key/value latent
  const T* kv = row + q_rank;
  float s2 = 0.f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = to_f32(kv[i]); s2 += v * v; }
  s2 = block_sum(s2, red);
  const float kinv = 1.0f / sqrtf(s2 / (float)kv_rank + eps);
  const int slot = slot_mapping[t];
  if (slot < 0) return;                                 // a padding row: nothing is stored
  if (slot >= num_slots) {
    if (threadIdx.x == 0) report_error(err, PHOTON_DEV_BAD_SLOT, t, slot, (int)num_slots);
    return;
  }
  T* dst = cache + (size_t)slot * (kv_rank + rot);
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x)
    dst[i] = from_f32<T>(to_f32(kv[i]) * kinv * load_w(kw, kw_bf16, i));
  const T* kr = kv + kv_rank;
  const int half = rot_dims / 2;
  const float p = (float)positions[t];
  for (int i = threadIdx.x; i < rot; i += blockDim.x) {
    float y;
    if (i < half) {
      float sn, cs;
      sincosf(p * inv_freq[i], &sn, &cs);
      y = to_f32(kr[i]) * cs - to_f32(kr[i + half]) * sn;
    } else if (i < rot_dims) {
      float sn, cs;
      sincosf(p * inv_freq[i - half], &sn, &cs);
      y = to_f32(kr[i]) * cs + to_f32(kr[i - half]) * sn;
    } else {
      y = to_f32(kr[i]);
    }
    dst[kv_rank + i] = from_f32<T>(y);
  }
}

// down [T][q_rank + kv_rank + rot] (row stride in elements): the fused down-projections of a token.
// cq [T][q_rank]: the normed query latent.  cache: [num_slots][kv_rank + rot], the pages of one layer.
PHOTON_API int photon_latent_prep(const void* down, long down_stride, int dtype, int q_rank, int kv_rank, int rot,
                                  int rot_dims, const void* q_norm_w, int q_norm_dtype, const void* kv_norm_w,
                                  int kv_norm_dtype, float eps, const int* positions, const float* inv_freq,
                                  const int* slot_mapping, void* cq, long cq_stride, void* cache, long num_slots,
                                  int T_, int* err, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (q_rank <= 0 || kv_rank <= 0 || rot < 0 || rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return PHOTON_ERR_ARGUMENT;
  const int threads = 128;
  if (dtype == PHOTON_BF16)
    latent_prep_kernel<bf16><<<T_, threads, 0, stream>>>((const bf16*)down, down_stride, q_rank, kv_rank, rot, rot_dims,
        q_norm_w, q_norm_dtype == PHOTON_BF16, kv_norm_w, kv_norm_dtype == PHOTON_BF16, eps, positions, inv_freq,
        slot_mapping, (bf16*)cq, cq_stride, (bf16*)cache, num_slots, err);
  else
    latent_prep_kernel<float><<<T_, threads, 0, stream>>>((const float*)down, down_stride, q_rank, kv_rank, rot, rot_dims,
        q_norm_w, q_norm_dtype == PHOTON_BF16, kv_norm_w, kv_norm_dtype == PHOTON_BF16, eps, positions, inv_freq,
        slot_mapping, (float*)cq, cq_stride, (float*)cache, num_slots, err);
  return launch_status();
}

// ---------------------------------------------------------------- rotated query parts
// q [T][heads][dim + rot] -> out [T][heads][out_head] at offset out_off: the last rot numbers of every head, rotated.
template <typename T>
__global__ void latent_q_rope_kernel(const T* __restrict__ q, long q_stride, int heads, int dim, int rot, int rot_dims,
                                     const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                     T* __restrict__ out, long out_stride, int out_head, int out_off) {
  const int t = blockIdx.x;
  const float p = (float)positions[t];
  const int half = rot_dims / 2;
  for (int idx = threadIdx.x; idx < heads * rot; idx += blockDim.x) {
    const int h = idx / rot, i = idx - h * rot;
    const T* src = q + (size_t)t * q_stride + (size_t)h * (dim + rot) + dim;
    float y;
    if (i < half) {
      float sn, cs;
      sincosf(p * inv_freq[i], &sn, &cs);
      y = to_f32(src[i]) * cs - to_f32(src[i + half]) * sn;
    } else if (i < rot_dims) {
      float sn, cs;
      sincosf(p * inv_freq[i - half], &sn, &cs);
      y = to_f32(src[i]) * cs + to_f32(src[i - half]) * sn;
    } else {
      y = to_f32(src[i]);
    }
    out[(size_t)t * out_stride + (size_t)h * out_head + out_off + i] = from_f32<T>(y);
  }
}

PHOTON_API int photon_latent_q_rope(const void* q, long q_stride, int dtype, int heads, int dim, int rot, int rot_dims,
                                    const int* positions, const float* inv_freq, void* out, long out_stride,
                                    int out_head, int out_off, int T_, cudaStream_t stream) {
  if (T_ <= 0 || rot <= 0) return 0;
  if (rot_dims < 0 || rot_dims > rot || (rot_dims & 1)) return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_BF16)
    latent_q_rope_kernel<bf16><<<T_, 128, 0, stream>>>((const bf16*)q, q_stride, heads, dim, rot, rot_dims, positions,
                                                      inv_freq, (bf16*)out, out_stride, out_head, out_off);
  else
    latent_q_rope_kernel<float><<<T_, 128, 0, stream>>>((const float*)q, q_stride, heads, dim, rot, rot_dims, positions,
                                                       inv_freq, (float*)out, out_stride, out_head, out_off);
  return launch_status();
}

// ---------------------------------------------------------------- one product per head
// out[t, h, n] = sum_k x[t, h, k] * W[h, n, k], accumulated in 32-bit as one chain of K fused multiply-adds in
// ascending k (a row's result depends on nothing but the row).  Tiles of 64 tokens x 64 features per block.
#define HL_BM 64
#define HL_BN 64
#define HL_BK 16

template <typename T>
__global__ void __launch_bounds__(256)
head_linear_kernel(const T* __restrict__ x, long x_row, long x_head, const T* __restrict__ W, T* __restrict__ out,
                   long o_row, long o_head, int M, int N, int K) {
  __shared__ float As[HL_BK][HL_BM + 4];
  __shared__ float Ws[HL_BK][HL_BN + 4];
  const int h = blockIdx.z;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * HL_BM, n0 = blockIdx.x * HL_BN;
  const T* A = x + (size_t)h * x_head;
  const T* Wh = W + (size_t)h * N * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HL_BK) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const int idx = tid + r * 256;
      const int row = idx >> 4, kk = idx & 15;
      const int gm = m0 + row, gn = n0 + row, gk = k0 + kk;
      As[kk][row] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * x_row + gk]) : 0.f;
      Ws[kk][row] = (gn < N && gk < K) ? to_f32(Wh[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < HL_BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) out[(size_t)gm * o_row + (size_t)h * o_head + gn] = from_f32<T>(acc[i][j]);
    }
  }
}

// Few bfloat16 rows (decode steps): the rows of x of one head wait in shared memory, every warp streams four rows
// of W[h] once, 16 bytes per lane and load, against all of them.
#define HLS_ROWS 8
__global__ void __launch_bounds__(256)
head_linear_skinny_kernel(const bf16* __restrict__ x, long x_row, long x_head, const bf16* __restrict__ W,
                          bf16* __restrict__ out, long o_row, long o_head, int M, int N, int K) {
  extern __shared__ __align__(16) bf16 xs[];                 // M x K
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x * 8; i < M * K; i += blockDim.x * 8) {
    const int m = i / K, k = i - m * K;
    *reinterpret_cast<uint4*>(xs + i) = *reinterpret_cast<const uint4*>(x + (size_t)m * x_row + (size_t)h * x_head + k);
  }
  __syncthreads();
  const bf16* Wh = W + (size_t)h * N * K;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const int n = blockIdx.x * 32 + c * 8 + warp;
    if (n >= N) continue;
    float acc[HLS_ROWS];
#pragma unroll
    for (int m = 0; m < HLS_ROWS; ++m) acc[m] = 0.f;
    for (int k = lane * 8; k < K; k += 256) {
      const uint4 wv = *reinterpret_cast<const uint4*>(Wh + (size_t)n * K + k);
      const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
      float wf[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(wp[i]); wf[2 * i] = f.x; wf[2 * i + 1] = f.y; }
#pragma unroll
      for (int m = 0; m < HLS_ROWS; ++m) {
        if (m < M) {
          const uint4 xv = *reinterpret_cast<const uint4*>(xs + m * K + k);
          const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(xp[i]);
            acc[m] = fmaf(f.x, wf[2 * i], acc[m]);
            acc[m] = fmaf(f.y, wf[2 * i + 1], acc[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < HLS_ROWS; ++m) {
      if (m < M) {
        const float v = warp_sum(acc[m]);
        if (lane == 0) out[(size_t)m * o_row + (size_t)h * o_head + n] = __float2bfloat16_rn(v);
      }
    }
  }
}

// x [M][heads][K] and out [M][heads][N] with row and head strides in elements; W [heads][N][K] contiguous.
PHOTON_API int photon_head_linear(const void* x, long x_row, long x_head, const void* W, void* out, long o_row,
                                  long o_head, int dtype, int M, int heads, int N, int K, cudaStream_t stream) {
  if (M <= 0 || heads <= 0 || N <= 0) return 0;
  if (K <= 0) return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_BF16 && M <= HLS_ROWS && K % 8 == 0 && x_row % 8 == 0 && x_head % 8 == 0 && (uintptr_t)x % 16 == 0 &&
      (uintptr_t)W % 16 == 0 && heads <= 65535 && (size_t)M * K * 2 <= 48 * 1024) {
    head_linear_skinny_kernel<<<dim3((N + 31) / 32, heads), 256, (size_t)M * K * 2, stream>>>(
        (const bf16*)x, x_row, x_head, (const bf16*)W, (bf16*)out, o_row, o_head, M, N, K);
    return launch_status();
  }
  dim3 grid((N + HL_BN - 1) / HL_BN, (M + HL_BM - 1) / HL_BM, heads);
  if (grid.y > 65535 || grid.z > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (dtype == PHOTON_BF16)
    head_linear_kernel<bf16><<<grid, 256, 0, stream>>>((const bf16*)x, x_row, x_head, (const bf16*)W, (bf16*)out, o_row,
                                                      o_head, M, N, K);
  else
    head_linear_kernel<float><<<grid, 256, 0, stream>>>((const float*)x, x_row, x_head, (const float*)W, (float*)out,
                                                       o_row, o_head, M, N, K);
  return launch_status();
}

// ---------------------------------------------------------------- a request's cached rows, in order
// out[p, :] = cache[table[p / page_size] * page_size + p % page_size, :] for p < count: the latent rows of one
// request as one dense matrix, the operand of the products that attention over a long prompt portion is made of.
template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ cache, const int* __restrict__ table, int page_size,
                                   int num_pages, int width, int count, T* __restrict__ out, int* err) {
  const int p = blockIdx.x;
  const int page = table[p / page_size];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) report_error(err, PHOTON_DEV_BAD_PAGE, 0, p, page);
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)p * width + i] = from_f32<T>(0.f);
    return;
  }
  const T* src = cache + ((size_t)page * page_size + p % page_size) * width;
  for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)p * width + i] = src[i];
}

PHOTON_API int photon_gather_rows(const void* cache, int dtype, const int* table, int page_size, int num_pages,
                                  int width, int count, void* out, int* err, cudaStream_t stream) {
  if (count <= 0) return 0;
  if (page_size <= 0 || width <= 0) return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_BF16)
    gather_rows_kernel<bf16><<<count, 128, 0, stream>>>((const bf16*)cache, table, page_size, num_pages, width, count, (bf16*)out, err);
  else
    gather_rows_kernel<float><<<count, 128, 0, stream>>>((const float*)cache, table, page_size, num_pages, width, count, (float*)out, err);
  return launch_status();
}

// ---------------------------------------------------------------- causal softmax over rows of scores
// scores [rows][ld] float: row r belongs to the token at position first_pos + r / heads, which sees the keys
// 0 .. its own position.  probs [rows][ldp] = softmax(scale * scores) over the visible keys, zero beyond them, up to
// column `cols`.  One block per row, 32-bit throughout, rounded once on the way out.
template <typename T>
__global__ void causal_softmax_kernel(const float* __restrict__ scores, long ld, T* __restrict__ probs, long ldp,
                                      int heads, int first_pos, int cols, float scale) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int visible = min(cols, first_pos + r / heads + 1);
  const float* s = scores + (size_t)r * ld;
  T* p = probs + (size_t)r * ldp;
  float m = -INFINITY;
  for (int i = threadIdx.x; i < visible; i += blockDim.x) m = fmaxf(m, s[i] * scale);
  m = warp_max(m);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : -INFINITY;
  m = warp_max(m);
  float sum = 0.f;
  for (int i = threadIdx.x; i < visible; i += blockDim.x) sum += expf(s[i] * scale - m);
  sum = block_sum(sum, red);
  const float inv = 1.0f / sum;
  for (int i = threadIdx.x; i < cols; i += blockDim.x)
    p[i] = from_f32<T>(i < visible ? expf(s[i] * scale - m) * inv : 0.f);
}

PHOTON_API int photon_causal_softmax_rows(const float* scores, long ld, void* probs, long ldp, int dtype, int rows,
                                          int heads, int first_pos, int cols, float scale, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if (heads <= 0 || first_pos < 0) return PHOTON_ERR_ARGUMENT;
  if (dtype == PHOTON_BF16)
    causal_softmax_kernel<bf16><<<rows, 256, 0, stream>>>(scores, ld, (bf16*)probs, ldp, heads, first_pos, cols, scale);
  else
    causal_softmax_kernel<float><<<rows, 256, 0, stream>>>(scores, ld, (float*)probs, ldp, heads, first_pos, cols, scale);
  return launch_status();
}

// ---------------------------------------------------------------- decoded tokens on the tensor cores
// All heads of a token attend to the same cached rows, so a decoded token is a (heads x width) by (width x keys)
// product followed by a (heads x keys) by (keys x kv_rank) one.  Block (t, s) takes token t and the 64 keys
// s * 64 .. of its request: the rows come into shared memory once (16-byte loads through the block table) and
// serve every tile of 16 heads; scores = Q C^T with wmma (bfloat16 in, 32-bit accumulate), a softmax over the
// block's keys in 32-bit, P (rounded to bfloat16) times the first kv_rank columns of the same rows.  Every block
// leaves its unnormalised sums with the rows' maximum and denominator, in the layout of the general kernel's
// shares, and a second kernel puts the shares of a (token, head) together in their order.
#include <mma.h>
using namespace nvcuda;

#define LD_KEYS 64

__global__ void __launch_bounds__(128)
latent_decode_kernel(const bf16* __restrict__ q, long q_stride, const bf16* __restrict__ cache,
                     const int* __restrict__ block_table, int max_pages, const int* __restrict__ token_seq,
                     const int* __restrict__ positions, int heads, int width, int dv, int page_size, int num_pages,
                     float scale, int splits, float* __restrict__ part, int* err) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int t = blockIdx.x, s = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ldk = width + 8;                                   // bfloat16 elements; rows of 16 keys stay 32-byte aligned
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw);                // 64 x ldk
  bf16* Qs = Ks + LD_KEYS * ldk;                               // 16 x ldk
  float* Sf = reinterpret_cast<float*>(Qs + 16 * ldk);         // 16 x 68
  bf16* Ps = reinterpret_cast<bf16*>(Sf + 16 * 68);            // 16 x 72
  float* Ot = reinterpret_cast<float*>(Ps + 16 * 72);          // 4 x 16 x 20
  float* rowm = Ot + 4 * 16 * 20;                              // 16
  float* rowl = rowm + 16;                                     // 16
  const int p = positions[t];
  const int k0 = s * LD_KEYS;
  const int nkeys = min(LD_KEYS, p + 1 - k0);                  // keys of this block that the token sees
  if (nkeys <= 0) {                                            // an empty share: the merge skips it
    for (int h = tid; h < heads; h += 128) {
      float* dst = part + (((size_t)t * heads + h) * splits + s) * (dv + 2);
      dst[dv] = -INFINITY; dst[dv + 1] = 0.f;
    }
    return;
  }
  const int* table = block_table + (size_t)token_seq[t] * max_pages;
  const int vecs = width / 8;
  // where each of the block's rows lies, looked up once; the loads of the rows then depend on nothing but this list
  long long* rowbase = reinterpret_cast<long long*>(rowl + 16);
  if (tid < LD_KEYS) {
    long long base = -1;
    if (tid < nkeys) {
      const int kk = k0 + tid;
      const int page = table[kk / page_size];
      if (page < 0 || page >= num_pages) report_error(err, PHOTON_DEV_BAD_PAGE, t, kk, page);
      else base = ((long long)page * page_size + kk % page_size) * width;
    }
    rowbase[tid] = base;
  }
  __syncthreads();
#pragma unroll 4
  for (int i = tid; i < LD_KEYS * vecs; i += 128) {
    const int key = i / vecs, j = (i - key * vecs) * 8;
    const long long base = rowbase[key];
    uint4 raw = make_uint4(0, 0, 0, 0);
    if (base >= 0) raw = *reinterpret_cast<const uint4*>(cache + base + j);
    *reinterpret_cast<uint4*>(Ks + key * ldk + j) = raw;
  }
  for (int h0 = 0; h0 < heads; h0 += 16) {
    __syncthreads();                                           // the rows are in; the last tile of heads is done with Qs
    for (int i = tid; i < 16 * vecs; i += 128) {
      const int h = i / vecs, j = (i - h * vecs) * 8;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (h0 + h < heads) raw = *reinterpret_cast<const uint4*>(q + (size_t)t * q_stride + (size_t)(h0 + h) * width + j);
      *reinterpret_cast<uint4*>(Qs + h * ldk + j) = raw;
    }
    __syncthreads();
    {   // scores of 16 heads x 16 keys per warp
      wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
      wmma::fill_fragment(acc, 0.f);
      for (int k = 0; k < width; k += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::col_major> b;
        wmma::load_matrix_sync(a, Qs + k, ldk);
        wmma::load_matrix_sync(b, Ks + (size_t)warp * 16 * ldk + k, ldk);
        wmma::mma_sync(acc, a, b, acc);
      }
      wmma::store_matrix_sync(Sf + warp * 16, acc, 68, wmma::mem_row_major);
    }
    __syncthreads();
    {   // softmax over the block's keys: eight lanes a row, eight keys a lane
      const int row = tid >> 3, c0 = (tid & 7) * 8;
      float v[8], m = -INFINITY;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        v[u] = c0 + u < nkeys ? Sf[row * 68 + c0 + u] * scale : -INFINITY;
        m = fmaxf(m, v[u]);
      }
      for (int d = 1; d < 8; d <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      float l = 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const float e = v[u] == -INFINITY ? 0.f : expf(v[u] - m);
        l += e;
        Ps[row * 72 + c0 + u] = __float2bfloat16_rn(e);
      }
      for (int d = 1; d < 8; d <<= 1) l += __shfl_xor_sync(0xffffffffu, l, d);
      if ((tid & 7) == 0) { rowm[row] = m; rowl[row] = l; }
    }
    __syncthreads();
    for (int nt = warp; nt < dv / 16; nt += 4) {               // 16 heads x 16 value columns per tile
      wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc;
      wmma::fill_fragment(acc, 0.f);
#pragma unroll
      for (int kk = 0; kk < LD_KEYS; kk += 16) {
        wmma::fragment<wmma::matrix_a, 16, 16, 16, bf16, wmma::row_major> a;
        wmma::fragment<wmma::matrix_b, 16, 16, 16, bf16, wmma::row_major> b;
        wmma::load_matrix_sync(a, Ps + kk, 72);
        wmma::load_matrix_sync(b, Ks + (size_t)kk * ldk + nt * 16, ldk);
        wmma::mma_sync(acc, a, b, acc);
      }
      float* stage = Ot + warp * 16 * 20;
      wmma::store_matrix_sync(stage, acc, 20, wmma::mem_row_major);
      __syncwarp();
      for (int e = lane; e < 256; e += 32) {
        const int h = e >> 4, c = e & 15;
        if (h0 + h < heads)
          part[(((size_t)t * heads + h0 + h) * splits + s) * (dv + 2) + nt * 16 + c] = stage[h * 20 + c];
      }
      __syncwarp();
    }
    if (tid < 16 && h0 + tid < heads) {
      float* dst = part + (((size_t)t * heads + h0 + tid) * splits + s) * (dv + 2);
      dst[dv] = rowm[tid]; dst[dv + 1] = rowl[tid];
    }
  }
}

__global__ void latent_merge_kernel(const float* __restrict__ part, int splits, int dv, bf16* __restrict__ out,
                                    long out_stride, int heads) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float* src = part + ((size_t)t * heads + h) * splits * (dv + 2);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, src[s * (dv + 2) + dv]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = src[s * (dv + 2) + dv];
    if (ms != -INFINITY) l += src[s * (dv + 2) + dv + 1] * expf(ms - m);
  }
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = src[s * (dv + 2) + dv];
      if (ms != -INFINITY) a += src[s * (dv + 2) + j] * expf(ms - m);
    }
    out[(size_t)t * out_stride + (size_t)h * dv + j] = __float2bfloat16_rn(l > 0.f ? a / l : 0.f);
  }
}

// q [T][heads * width] bfloat16 (row stride in elements), cache [num_pages * page_size][width] bfloat16, out
// [T][heads * dv]: token t at position positions[t] of request token_seq[t] sees the rows 0 .. positions[t]; a row's
// value is its first dv numbers.  width and dv multiples of 16.  splits >= ceil((largest position + 1) / 64);
// part: float [T * heads * splits * (dv + 2)].
PHOTON_API int photon_latent_decode_attention(const void* q, long q_stride, const void* cache, const int* block_table,
                                              int max_pages, const int* token_seq, const int* positions, int T_,
                                              int heads, int width, int dv, int page_size, int num_pages, float scale,
                                              int splits, float* part, void* out, long out_stride, int* err,
                                              cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (heads <= 0 || splits <= 0 || part == nullptr || dv > width) return PHOTON_ERR_ARGUMENT;
  if (width % 16 || dv % 16 || q_stride % 8 || (uintptr_t)q % 16 || (uintptr_t)cache % 16 || splits > 65535 || heads > 65535)
    return PHOTON_ERR_UNSUPPORTED;
  const size_t smem = (size_t)(LD_KEYS + 16) * (width + 8) * 2 + 16 * 68 * 4 + 16 * 72 * 2 + 4 * 16 * 20 * 4 + 32 * 4 + LD_KEYS * 8;
  if (smem > 220 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(latent_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  latent_decode_kernel<<<dim3(T_, splits), 128, smem, stream>>>((const bf16*)q, q_stride, (const bf16*)cache, block_table,
      max_pages, token_seq, positions, heads, width, dv, page_size, num_pages, scale, splits, part, err);
  int st = launch_status();
  if (st != 0) return st;
  latent_merge_kernel<<<dim3(T_, heads), 128, 0, stream>>>(part, splits, dv, (bf16*)out, out_stride, heads);
  return launch_status();
}
