// Paged causal attention with grouped heads, the general kernel: any head size that
// is even, any number of heads and groups, any page size, float or bfloat16 storage,
// an optional window.  One block handles one token of the step and one key/value head
// (all query heads of that group), walks the keys in tiles of 32 from the cache and
// keeps a running softmax in 32-bit.  Prompt portions and single decoded tokens are
// the same case: a token at position p of its request sees the keys
// max(0, p - window + 1) .. p, which the cache holds once this step's keys are written.
//
// Formula: include/photon/ops/kernels/mha_kernel.hpp:188-229 (scores (q.k)/sqrt(d) for
// keys <= pos only, softmax exp(s - max)/sum, weighted sum of values; query head h
// uses key/value head h / (n_q / n_kv)).  The reference's paged kernel
// (src/ops/kernels/cuda/paged_attention.cu:90-194) adds 1e-6 to the denominator and
// lets a token see later tokens of its own portion; neither is done here.
//
// The tile grid starts at key 0 (at a multiple of 32 at or below the window's first
// key), so the order of every sum depends only on the token's position, never on how
// the request was cut into steps or on what else is in the batch.
//
// Two generalisations serve mixers whose keys and values are not two tensors of one head size.  The value of
// a key is `dv` numbers wide (dv <= d); with v_cache == k_cache the value is the first dv numbers of the key's
// own row (attention over a cached latent: the latent is key and value at once, the rest of the row is a
// rotated key part).  And the query heads that share a key/value head are cut into chunks of `hb` heads per
// block, so that any number of query heads may share one key/value head.
#include "common.cuh"
#include <math.h>

#define ATT_TILE 32
#define ATT_THREADS 128

template <typename T, int PPT>
__global__ void __launch_bounds__(ATT_THREADS)
paged_attention_kernel(const T* __restrict__ q, long q_stride, T* __restrict__ out, long out_stride,
                       const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       const int* __restrict__ block_table, int max_pages,
                       const int* __restrict__ token_seq, const int* __restrict__ positions,
                       int n_q, int n_kv, int d, int dv, int hb, int page_size, int num_pages, int window,
                       float scale, int splits, float* __restrict__ part, int* err, int keep_first, int sink,
                       float softcap, const T* __restrict__ gate, long gate_stride) {
  extern __shared__ __align__(16) float smem[];
  const int chunks = (n_q / n_kv + hb - 1) / hb;
  const int t = blockIdx.x, g = blockIdx.y / chunks;
  const int h0 = g * (n_q / n_kv) + (blockIdx.y % chunks) * hb;            // first query head of this block
  const int G = min(hb, (g + 1) * (n_q / n_kv) - h0);                      // query heads of this block
  const bool shared_kv = (const void*)v_cache == (const void*)k_cache;    // values are the head of the key rows
  const int vld = shared_kv ? d + 1 : dv;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* qs = smem;                          // G * d
  float* ks = qs + hb * d;                   // TILE * (d + 1)
  float* vs = ks + ATT_TILE * (d + 1);       // TILE * dv (not used when the values lie in the key rows)
  float* sc = vs + (shared_kv ? 0 : ATT_TILE * dv);   // hb * TILE
  float* mrun = sc + hb * ATT_TILE;          // hb
  float* lsum = mrun + hb;                   // hb
  float* corr = lsum + hb;                   // hb
  long long* kbase = (long long*)(corr + hb + ((hb & 1) ? 1 : 0));   // TILE (8-byte aligned)
  if (shared_kv) vs = ks;

  const int p = positions[t];
  const int seq = token_seq[t];
  const int kstart = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int* table = block_table + (size_t)seq * max_pages;

  {
    // the block's query heads lie side by side in the row: 16 bytes per load where the row allows it
    constexpr int QV = 16 / sizeof(T);
    const T* qrow = q + (size_t)t * q_stride + (size_t)h0 * d;
    if ((G * d) % QV == 0 && (uintptr_t)qrow % 16 == 0) {
      for (int i = tid * QV; i < G * d; i += ATT_THREADS * QV) {
        const uint4 raw = *reinterpret_cast<const uint4*>(qrow + i);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int u = 0; u < QV; ++u) qs[i + u] = to_f32(e[u]);
      }
    } else {
      for (int i = tid; i < G * d; i += ATT_THREADS) qs[i] = to_f32(qrow[i]);
    }
  }
  for (int h = tid; h < G; h += ATT_THREADS) { mrun[h] = -INFINITY; lsum[h] = 0.f; corr[h] = 0.f; }
  float acc[PPT];
#pragma unroll
  for (int n = 0; n < PPT; ++n) acc[n] = 0.f;

  // the key tiles of this block: all of them, or one of `splits` equal shares (blockIdx.z)
  // With a window and kept first keys the walk has two stretches: the tiles of keys 0 .. keep_first - 1 that lie
  // below the window's first tile, then the window's tiles.  vt counts through both.
  const int tile_lo = kstart / ATT_TILE, tile_hi = p / ATT_TILE + 1;
  const int kept_tiles = (keep_first > 0 && kstart > 0) ? min((keep_first + ATT_TILE - 1) / ATT_TILE, tile_lo) : 0;
  int vt_lo = 0, vt_hi = kept_tiles + tile_hi - tile_lo;
  if (splits > 1) {
    const int per = (vt_hi + splits - 1) / splits;
    vt_lo = blockIdx.z * per;
    vt_hi = min(vt_hi, vt_lo + per);
  }
  constexpr int VEC = 16 / sizeof(T);
  const bool vec = (d % VEC == 0) && ((uintptr_t)k_cache % 16 == 0);
  for (int vt = vt_lo; vt < vt_hi; ++vt) {
    const int tile0 = (vt < kept_tiles ? vt : tile_lo + vt - kept_tiles) * ATT_TILE;
    __syncthreads();                          // previous tile fully consumed; qs ready on the first pass
    if (tid < ATT_TILE) {
      const int kk = tile0 + tid;
      long long base = -1;
      if (kk <= p && (kk >= kstart || kk < keep_first)) {
        const int page = table[kk / page_size];
        if (page < 0 || page >= num_pages) {
          report_error(err, PHOTON_DEV_BAD_PAGE, t, kk, page);
        } else {
          base = (((long long)page * n_kv + g) * page_size + (kk % page_size)) * d;
        }
      }
      kbase[tid] = base;
    }
    __syncthreads();
    if (vec) {
      const int per_key = d / VEC;
#pragma unroll 4
      for (int i = tid; i < ATT_TILE * per_key; i += ATT_THREADS) {
        const int key = i / per_key, j = (i - key * per_key) * VEC;
        const long long base = kbase[key];
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (base >= 0) raw = *reinterpret_cast<const uint4*>(k_cache + base + j);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int u = 0; u < VEC; ++u) ks[key * (d + 1) + j + u] = to_f32(e[u]);
      }
    } else {
      for (int i = tid; i < ATT_TILE * d; i += ATT_THREADS) {
        const int key = i / d, j = i - key * d;
        const long long base = kbase[key];
        ks[key * (d + 1) + j] = base >= 0 ? to_f32(k_cache[base + j]) : 0.f;
      }
    }
    if (!shared_kv) {
      for (int i = tid; i < ATT_TILE * dv; i += ATT_THREADS) {
        const int key = i / dv, j = i - key * dv;
        const long long base = kbase[key];
        vs[key * dv + j] = base >= 0 ? to_f32(v_cache[base / d * dv + j]) : 0.f;
      }
    }
    __syncthreads();
    // scores
    for (int i = tid; i < G * ATT_TILE; i += ATT_THREADS) {
      const int h = i / ATT_TILE, key = i - h * ATT_TILE;
      float s = -INFINITY;
      if (kbase[key] >= 0) {
        const float* qh = qs + h * d;
        const float* kr = ks + key * (d + 1);
        float dot = 0.f;
        for (int j = 0; j < d; ++j) dot += qh[j] * kr[j];
        s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
      }
      sc[i] = s;
    }
    __syncthreads();
    // running softmax, one warp per head, one lane per key of the tile
    for (int h = warp; h < G; h += ATT_THREADS / 32) {
      const float s = sc[h * ATT_TILE + lane];
      const float tmax = warp_max(s);
      const float m_old = mrun[h];
      const float m_new = fmaxf(m_old, tmax);
      const float pr = (s == -INFINITY) ? 0.f : expf(s - m_new);
      const float psum = warp_sum(pr);
      const float c = (m_old == -INFINITY) ? 0.f : expf(m_old - m_new);
      __syncwarp();
      sc[h * ATT_TILE + lane] = pr;
      if (lane == 0) { mrun[h] = m_new; lsum[h] = lsum[h] * c + psum; corr[h] = c; }
    }
    __syncthreads();
    // weighted values
#pragma unroll
    for (int n = 0; n < PPT; ++n) {
      const int i = tid + n * ATT_THREADS;
      if (i < G * dv) {
        const int h = i / dv, j = i - h * dv;
        float a = acc[n] * corr[h];
        const float* pr = sc + h * ATT_TILE;
#pragma unroll 8
        for (int key = 0; key < ATT_TILE; ++key) a += pr[key] * vs[key * vld + j];
        acc[n] = a;
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int n = 0; n < PPT; ++n) {
    const int i = tid + n * ATT_THREADS;
    if (i < G * dv) {
      const int h = i / dv, j = i - h * dv;
      float l = lsum[h];
      // the sink: one more key with score 0 and no value (only the denominator grows)
      if (sink && splits <= 1) l += expf(-mrun[h]);
      if (splits > 1) {
        // this share's sums as they stand, with the head's running maximum and denominator behind them
        float* dst = part + (((size_t)t * n_q + h0 + h) * splits + blockIdx.z) * (dv + 2);
        dst[j] = acc[n];
        if (j == 0) { dst[dv] = mrun[h]; dst[dv + 1] = l; }
      } else {
        float y = l > 0.f ? acc[n] / l : 0.f;
        if (gate) y = y / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + (size_t)(h0 + h) * dv + j])));
        out[(size_t)t * out_stride + (size_t)(h0 + h) * dv + j] = from_f32<T>(y);
      }
    }
  }
}

// The shares of one (token, head) put together, in the order of the shares.
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part, int splits, int dv, T* __restrict__ out,
                                       long out_stride, int n_q, int sink, const T* __restrict__ gate, long gate_stride) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float* src = part + ((size_t)t * n_q + h) * splits * (dv + 2);
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, src[s * (dv + 2) + dv]);
  float l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = src[s * (dv + 2) + dv];
    if (ms != -INFINITY) l += src[s * (dv + 2) + dv + 1] * expf(ms - m);
  }
  if (sink) l += expf(-m);
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = src[s * (dv + 2) + dv];
      if (ms != -INFINITY) a += src[s * (dv + 2) + j] * expf(ms - m);
    }
    float y = l > 0.f ? a / l : 0.f;
    if (gate) y = y / (1.0f + expf(-to_f32(gate[(size_t)t * gate_stride + (size_t)h * dv + j])));
    out[(size_t)t * out_stride + (size_t)h * dv + j] = from_f32<T>(y);
  }
}

template <typename T, int PPT>
static int attention_launch(const void* q, long q_stride, void* out, long out_stride, const void* k_cache,
                            const void* v_cache, const int* block_table, int max_pages, const int* token_seq,
                            const int* positions, int T_, int n_q, int n_kv, int d, int dv, int hb, int page_size,
                            int num_pages, int window, float scale, int splits, float* part, int* err,
                            cudaStream_t stream, int keep_first, int sink, float softcap, const void* gate,
                            long gate_stride) {
  const int G = hb;
  const size_t floats = (size_t)G * d + ATT_TILE * (d + 1) + (v_cache == k_cache ? 0 : ATT_TILE * dv) +
                        (size_t)G * ATT_TILE + 3 * G + 1;
  const size_t smem = floats * sizeof(float) + ATT_TILE * sizeof(long long) + 8;
  if (smem > 220 * 1024) return PHOTON_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(paged_attention_kernel<T, PPT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid(T_, n_kv * ((n_q / n_kv + hb - 1) / hb), splits);
  paged_attention_kernel<T, PPT><<<grid, ATT_THREADS, smem, stream>>>(
      (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_cache, (const T*)v_cache, block_table,
      max_pages, token_seq, positions, n_q, n_kv, d, dv, hb, page_size, num_pages, window, scale, splits, part, err,
      keep_first, sink, softcap, splits > 1 ? nullptr : (const T*)gate, gate_stride);
  int st = launch_status();
  if (st != 0 || splits <= 1) return st;
  attention_merge_kernel<T><<<dim3(T_, n_q), 128, 0, stream>>>(part, splits, dv, (T*)out, out_stride, n_q, sink, (const T*)gate, gate_stride);
  return launch_status();
}

#define ATT_DISPATCH(TYPE)                                                                              \
  if (ppt <= 1) return attention_launch<TYPE, 1>(ATT_ARGS);                                             \
  if (ppt <= 2) return attention_launch<TYPE, 2>(ATT_ARGS);                                             \
  if (ppt <= 4) return attention_launch<TYPE, 4>(ATT_ARGS);                                             \
  if (ppt <= 8) return attention_launch<TYPE, 8>(ATT_ARGS);                                             \
  if (ppt <= 16) return attention_launch<TYPE, 16>(ATT_ARGS);                                           \
  if (ppt <= 32) return attention_launch<TYPE, 32>(ATT_ARGS);                                           \
  return PHOTON_ERR_UNSUPPORTED;

#define ATT_ARGS q, q_stride, out, out_stride, k_cache, v_cache, block_table, max_pages, token_seq, \
                 positions, T_, n_q, n_kv, d, dv, hb, page_size, num_pages, window, scale, splits, part, err, stream, \
                 keep_first, sink, softcap, gate, gate_stride

// window <= 0: all keys.  Strides in elements.  The key cache holds [num_pages][n_kv][page_size][d], the value
// cache [num_pages][n_kv][page_size][dv]; v_cache == k_cache (dv <= d): a key's value is the head of its row.
// out [T][n_q * dv].  A block runs up to 4096 / max(d, dv) of the query heads that share a key/value head.
// splits > 1: the key tiles of every token are shared out over that many blocks (decoded tokens with long
// contexts, where one block per token and head chunk leaves the GPU empty); part: float scratch of
// T * n_q * splits * (dv + 2); a second kernel puts the shares together in their order.
PHOTON_API int photon_paged_attention(const void* q, long q_stride, void* out, long out_stride, int dtype,
                                      const void* k_cache, const void* v_cache, const int* block_table,
                                      int max_pages, const int* token_seq, const int* positions, int T_,
                                      int n_q, int n_kv, int d, int dv, int page_size, int num_pages, int window,
                                      float scale, int splits, float* part, int* err, cudaStream_t stream) {
  return photon_paged_attention_ex(q, q_stride, out, out_stride, dtype, k_cache, v_cache, block_table, max_pages, token_seq,
                                   positions, T_, n_q, n_kv, d, dv, page_size, num_pages, window, scale, splits, part, err,
                                   0, 0, 0.f, nullptr, 0, stream);
}

// The same with three more rules.  keep_first > 0 (with a window): keys 0 .. keep_first - 1 stay visible behind the
// window, at their true positions.  sink != 0: the softmax has one more key with score 0 and no value, so the
// weights of a row add up to less than one: p_j = exp(s_j) / (exp(0) + sum exp(s_i)).  softcap > 0: scores are
// bounded, s <- softcap * tanh(s / softcap), after the scale.  gate (may be null; the type of q, [T][n_q * dv] with row
// stride gate_stride): every output is multiplied by sigmoid(gate) before it is rounded.
PHOTON_API int photon_paged_attention_ex(const void* q, long q_stride, void* out, long out_stride, int dtype,
                                         const void* k_cache, const void* v_cache, const int* block_table,
                                         int max_pages, const int* token_seq, const int* positions, int T_,
                                         int n_q, int n_kv, int d, int dv, int page_size, int num_pages, int window,
                                         float scale, int splits, float* part, int* err, int keep_first, int sink,
                                         float softcap, const void* gate, long gate_stride, cudaStream_t stream) {
  if (T_ <= 0) return 0;
  if (keep_first < 0 || softcap < 0.f) return PHOTON_ERR_ARGUMENT;
  if (splits < 1 || splits > 64 || (splits > 1 && part == nullptr) || T_ > 65535 * 32) return PHOTON_ERR_ARGUMENT;
  if (splits > 1 && n_q > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (n_kv <= 0 || n_q % n_kv || d <= 0 || dv <= 0 || page_size <= 0) return PHOTON_ERR_ARGUMENT;
  if (v_cache == k_cache && dv > d) return PHOTON_ERR_ARGUMENT;
  if (d > 4096 || dv > 4096) return PHOTON_ERR_UNSUPPORTED;
  int hb = 4096 / (d > dv ? d : dv);
  if (hb > n_q / n_kv) hb = n_q / n_kv;
  if ((long)n_kv * ((n_q / n_kv + hb - 1) / hb) > 65535) return PHOTON_ERR_UNSUPPORTED;
  const int ppt = (hb * dv + ATT_THREADS - 1) / ATT_THREADS;
  if (n_kv > 65535) return PHOTON_ERR_UNSUPPORTED;
  if (dtype == PHOTON_BF16) { ATT_DISPATCH(bf16) }
  ATT_DISPATCH(float)
}
