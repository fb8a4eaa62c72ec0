// Attention over a paged cache of latents: every position keeps one vector [c ; kr] of
// C + R numbers shared by all heads, c a normalised low-rank latent from which keys and values
// would be projected, kr a rotated key part.  The query side absorbs the key projection
// (q_lat = W_uk^T q), so a head's score is (q_lat . c + q_rot . kr) * scale and its output the
// weighted sum of the latents themselves, projected to values afterwards.  Options: a sliding
// window (query at p sees p - window < j <= p) and a learned sink per head, a number that joins
// the softmax's denominator as exp(sink) with no key, no value and no scaling.
//
// Kernels: the preparation of a step's rows (two RMS norms with plain weights, the rotation of
// the shared key part, the write into the page slots), the rotation of the queries' rotated
// parts, and the attention itself.  Scores, softmax weights, angles and norms are 32-bit;
// T says how the cache and the outputs that feed matrix products are stored.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kKeys = 32;   // keys per tile, aligned to absolute positions: the sum's order does not depend on the cut

// ---- rows of a step: query latent, cached latent, rotated shared key ---------------------------
// proj [tokens, ld] floats: [0, Q) the query's low-rank projection, [Q, Q + C) the latent's,
// [Q + C, Q + C + R) the shared key part.  cq (T) = rmsnorm(first) * wq; the cache row of the
// token's slot = [rmsnorm(second) * wc ; rotate(third)].
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_prep_kernel(T* __restrict__ cq, T* __restrict__ cache,
                                                               const float* __restrict__ proj, int ld, int Q, int C,
                                                               int R, const T* __restrict__ wq, const T* __restrict__ wc,
                                                               const int* __restrict__ positions,
                                                               const float* __restrict__ inv_freq, int rot_dims,
                                                               const int* __restrict__ slots, long long n_slots,
                                                               float eps) {
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = proj + (size_t)t * ld;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < Q; i += kThreads) sq += row[i] * row[i];
  for (int i = threadIdx.x; i < C; i += kThreads) sc += row[Q + i] * row[Q + i];
  sq = block_sum(sq, scratch);
  sc = block_sum(sc, scratch);
  const float iq = 1.0f / sqrtf(sq / (float)Q + eps), ic = 1.0f / sqrtf(sc / (float)C + eps);
  for (int i = threadIdx.x; i < Q; i += kThreads) cq[(size_t)t * Q + i] = from_f32<T>(row[i] * iq * to_f32(wq[i]));
  if (cache == nullptr) return;
  const long long slot = slots[t];
  if (slot < 0 || slot >= n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  T* dst = cache + (size_t)slot * (C + R);
  for (int i = threadIdx.x; i < C; i += kThreads) dst[i] = from_f32<T>(row[Q + i] * ic * to_f32(wc[i]));
  const float pos = (float)positions[t];
  const int half = rot_dims / 2;
  const float* kr = row + Q + C;
  for (int i = threadIdx.x; i < R; i += kThreads) {
    float v = kr[i];
    if (i < rot_dims) {
      const int f = i < half ? i : i - half;
      const float ang = pos * inv_freq[f];
      const float cs = cosf(ang), sn = sinf(ang);
      float lo, hi;
      rope_rotate(kr[f], kr[f + half], cs, sn, lo, hi);
      v = i < half ? lo : hi;
    }
    dst[C + i] = from_f32<T>(v);
  }
}

// ---- the queries' rotated parts ---------------------------------------------------------------
// q (T) [tokens, heads, D + R] -> q_cat (float) [tokens, heads, C + R]: columns [C, C + R) get the
// rotated last R entries of each head (the first C columns are the absorbed product's).
template <typename T>
__global__ void __launch_bounds__(kThreads) latent_q_rope_kernel(float* __restrict__ q_cat, const T* __restrict__ q,
                                                                 int heads, int D, int R, int C,
                                                                 const int* __restrict__ positions,
                                                                 const float* __restrict__ inv_freq, int rot_dims) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = rot_dims / 2;
  for (int idx = threadIdx.x; idx < heads * R; idx += kThreads) {
    const int h = idx / R, i = idx % R;
    const T* src = q + ((size_t)t * heads + h) * (D + R) + D;
    float v = to_f32(src[i]);
    if (i < rot_dims) {
      const int f = i < half ? i : i - half;
      const float ang = pos * inv_freq[f];
      const float cs = cosf(ang), sn = sinf(ang);
      float lo, hi;
      rope_rotate(to_f32(src[f]), to_f32(src[f + half]), cs, sn, lo, hi);
      v = i < half ? lo : hi;
    }
    q_cat[((size_t)t * heads + h) * (C + R) + C + i] = v;
  }
}

// ---- attention ------------------------------------------------------------------------------------
// One CTA takes up to QT consecutive rows of one request with all heads: the tiles of keys it
// stages in shared memory serve every (row, head) pair.  A warp owns pairs; a lane owns a key of
// the tile for the scores and columns of the output for the weighted sum.  Running maximum, sum
// and output of a pair live in shared memory; the sink opens them (maximum = sink, sum = 1).
struct LatentParams {
  void* out;              // [tokens, heads * C] of T
  const float* q;         // [tokens, heads, C + R]
  const void* cache;      // [pages * page_size, C + R] of T
  const float* sink;      // [heads] or null
  const int* q_start;
  const int* pos0;
  const int* block_table;
  int bt_width, heads, C, W, page_size, num_pages, window, QT;
  float scale;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) latent_attention_kernel(LatentParams p) {
  extern __shared__ float smem[];
  pdl_trigger();
  pdl_wait();
  const int req = blockIdx.y;
  const int first = p.q_start[req] + blockIdx.x * p.QT;
  const int n = min(p.QT, p.q_start[req + 1] - first);
  if (n <= 0) return;
  const int H = p.heads, C = p.C, W = p.W, KW = W + 1;
  const int pairs = n * H;
  float* qs = smem;                                  // [QT * H][W]
  float* keys = qs + (size_t)p.QT * H * W;           // [kKeys][W + 1]
  float* acc = keys + kKeys * KW;                    // [QT * H][C]
  float* run_m = acc + (size_t)p.QT * H * C;         // [QT * H]
  float* run_l = run_m + p.QT * H;
  float* probs = run_l + p.QT * H;                   // [kWarps][kKeys]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* cache = (const T*)p.cache;

  const int p_first = p.pos0[req] + blockIdx.x * p.QT, p_last = p_first + n - 1;
  const int lo = p.window > 0 ? max(0, p_first - p.window + 1) : 0;
  for (int i = tid; i < pairs * W; i += kThreads) qs[i] = p.q[(size_t)first * H * W + i];
  for (int i = tid; i < pairs * C; i += kThreads) acc[i] = 0.f;
  for (int i = tid; i < pairs; i += kThreads) {
    run_m[i] = p.sink != nullptr ? p.sink[i % H] : -INFINITY;
    run_l[i] = p.sink != nullptr ? 1.f : 0.f;
  }
  const int* table = p.block_table + (size_t)req * p.bt_width;

  for (int tile = lo / kKeys; tile <= p_last / kKeys; ++tile) {
    __syncthreads();       // the previous tile's readers are done (and the set-up above is visible)
    for (int jk = warp; jk < kKeys; jk += kWarps) {
      const int pos = tile * kKeys + jk;
      const T* src = nullptr;
      if (pos >= lo && pos <= p_last) {
        const int page = table[pos / p.page_size];
        if (page < 0 || page >= p.num_pages) {
          if (lane == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
        } else {
          src = cache + ((size_t)page * p.page_size + pos % p.page_size) * W;
        }
      }
      for (int c = lane; c < W; c += 32) keys[jk * KW + c] = src != nullptr ? to_f32(src[c]) : 0.f;
    }
    __syncthreads();
    for (int pair = warp; pair < pairs; pair += kWarps) {
      const int qpos = p_first + pair / H;
      const int kpos = tile * kKeys + lane;
      const bool seen = kpos <= qpos && kpos >= lo && (p.window <= 0 || qpos - kpos < p.window);
      float s = -INFINITY;
      if (seen) {
        const float* qv = qs + (size_t)pair * W;
        const float* kv = keys + lane * KW;
        float dot = 0.f;
        for (int c = 0; c < W; ++c) dot = fmaf(qv[c], kv[c], dot);
        s = dot * p.scale;
      }
      const float tile_max = warp_max(s);
      if (tile_max == -INFINITY) continue;           // the whole tile lies outside this row's reach
      const float m_old = run_m[pair];
      const float m_new = fmaxf(m_old, tile_max);
      const float corr = expf(m_old - m_new);        // m_old = -inf only without a sink: then 0
      const float pj = seen ? expf(s - m_new) : 0.f;
      const float sum = warp_sum(pj);
      __syncwarp();
      probs[warp * kKeys + lane] = pj;
      if (lane == 0) {
        run_m[pair] = m_new;
        run_l[pair] = run_l[pair] * corr + sum;
      }
      __syncwarp();
      const float* pw = probs + warp * kKeys;
      for (int c = lane; c < C; c += 32) {
        float a = acc[(size_t)pair * C + c] * corr;
#pragma unroll 8
        for (int jk = 0; jk < kKeys; ++jk) a = fmaf(pw[jk], keys[jk * KW + c], a);
        acc[(size_t)pair * C + c] = a;
      }
    }
  }
  __syncthreads();
  T* out = (T*)p.out + (size_t)first * H * C;
  for (int i = tid; i < pairs * C; i += kThreads) out[i] = from_f32<T>(acc[i] / run_l[i / C]);
}

size_t attention_smem(int QT, int H, int C, int W) {
  return sizeof(float) * ((size_t)QT * H * W + (size_t)kKeys * (W + 1) + (size_t)QT * H * C + 2 * (size_t)QT * H +
                          kWarps * kKeys);
}

}  // namespace

LAB_EXPORT int lab_latent_prep(void* cq, void* cache, const float* proj, int ld, int Q, int C, int R, const void* wq,
                               const void* wc, const int* positions, const float* inv_freq, int rot_dims,
                               const int* slots, long long n_slots, int tokens, float eps, int dtype,
                               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(latent_prep_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, (float*)cq, (float*)cache, proj, ld,
               Q, C, R, (const float*)wq, (const float*)wc, positions, inv_freq, rot_dims, slots, n_slots, eps);
  else
    lab_launch(latent_prep_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, (__nv_bfloat16*)cq,
               (__nv_bfloat16*)cache, proj, ld, Q, C, R, (const __nv_bfloat16*)wq, (const __nv_bfloat16*)wc, positions,
               inv_freq, rot_dims, slots, n_slots, eps);
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_latent_q_rope(float* q_cat, const void* q, int tokens, int heads, int D, int R, int C,
                                 const int* positions, const float* inv_freq, int rot_dims, int dtype,
                                 cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (dtype == LAB_F32)
    lab_launch(latent_q_rope_kernel<float>, dim3(tokens), dim3(kThreads), 0, stream, q_cat, (const float*)q, heads, D, R,
               C, positions, inv_freq, rot_dims);
  else
    lab_launch(latent_q_rope_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), 0, stream, q_cat,
               (const __nv_bfloat16*)q, heads, D, R, C, positions, inv_freq, rot_dims);
  LAB_LAUNCH_CHECK();
}

// Rows of a request that one CTA takes: as many (up to 8) as shared memory holds.
LAB_EXPORT int lab_latent_attention_rows(int heads, int C, int W, int max_q) {
  int qt = 8;
  while (qt > 1 && (attention_smem(qt, heads, C, W) > 96 * 1024 || qt / 2 >= max_q)) qt /= 2;
  if (attention_smem(qt, heads, C, W) > 200 * 1024) return 0;
  return qt;
}

LAB_EXPORT int lab_latent_attention(void* out, const float* q, const void* cache, const float* sink,
                                    const int* q_start, const int* pos0, const int* block_table, int bt_width,
                                    int n_requests, int max_q, int heads, int C, int W, int page_size, int num_pages,
                                    int window, float scale, int dtype, cudaStream_t stream) {
  if (n_requests <= 0 || max_q <= 0) return 0;
  LatentParams p;
  p.out = out; p.q = q; p.cache = cache; p.sink = sink; p.q_start = q_start; p.pos0 = pos0;
  p.block_table = block_table; p.bt_width = bt_width; p.heads = heads; p.C = C; p.W = W; p.page_size = page_size;
  p.num_pages = num_pages; p.window = window; p.scale = scale;
  p.QT = lab_latent_attention_rows(heads, C, W, max_q);
  if (p.QT <= 0) return (int)cudaErrorInvalidValue;
  const size_t smem = attention_smem(p.QT, heads, C, W);
  const dim3 grid((max_q + p.QT - 1) / p.QT, n_requests);
  cudaError_t e;
  if (dtype == LAB_F32) {
    e = cudaFuncSetAttribute(latent_attention_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lab_launch(latent_attention_kernel<float>, grid, dim3(kThreads), smem, stream, p);
  } else {
    e = cudaFuncSetAttribute(latent_attention_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return (int)e;
    lab_launch(latent_attention_kernel<__nv_bfloat16>, grid, dim3(kThreads), smem, stream, p);
  }
  LAB_LAUNCH_CHECK();
}
