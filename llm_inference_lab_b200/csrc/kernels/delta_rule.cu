// Generalized delta rule: a recurrent mixer whose state per head is a matrix S [key channel,
// value channel] in 32-bit floats, carried from token to token:
//
//   S <- diag(w) S  -  (a * u) (u^T S)  +  k v^T          (both products read the old S)
//   o  = S^T r
//
// with per-channel decay w = exp(-rate * sigmoid(d)), removal rate a = sigmoid(.), and the unit key
// u = k / sqrt(sum k^2 + 1e-6).  The kernel takes the projections r, k, v, the gate's and the two
// rates' pre-activations in 32-bit, forms every quantity of the recurrence in 32-bit, walks a
// request's tokens in order, divides each head's o by its root mean square, multiplies by a weight
// and by sigmoid(gate) and rounds to the storage type for the output projection.
//
// One CTA per (head, request, slice of CS columns of S).  Built per head size D (LAB_HEAD_DIM).  The
// columns of S are independent of one another, and so are its rows within a token, so a column is shared
// out over G threads (4 where D allows): thread g keeps the rows g * SL .. g * SL + SL - 1 of column j in
// registers, reads its share of each vector with consecutive 16-byte loads (a vector lies row block by
// row block with four floats of padding between the blocks, so the G threads of a column hit different
// banks, and lanes of other columns read the same addresses), and the sums over a column are finished by
// log2(G) shuffles.  (Blocks interleaved over the threads, without padding, are as free of conflicts and
// measured slower: 0.90 against 0.75 ms for 2,048 tokens of one request.)  What bounds the walk is the chain of dependent
// instructions one warp has per token (measured with the kernel's own clock: 540 cycles a token with
// 4 threads a column and 16 rows each), and a head's columns are shared out over D / CS CTAs so that
// no scheduler holds more than one such chain.  Tokens are taken in chunks:
// a chunk's records are brought to shared memory by cp.async into the buffer that is not being walked.
// Three kernels: a first one, parallel over tokens, forms what does not depend on the state (decays,
// rates, unit keys); the walk; a third, parallel over tokens, divides each head's raw output by its root
// mean square and applies weight and gate.  A step of one token per request (decode) is the same three
// kernels with a chunk of one.
#include "common.cuh"

#ifndef LAB_HEAD_DIM
#define LAB_HEAD_DIM 64
#endif

namespace {

constexpr int D = LAB_HEAD_DIM;
// threads per column: up to 4, so that every thread has whole blocks of four rows.  (Measured at D = 64,
// 2,048 tokens of one request: 4 threads a column 0.74 ms, 16 threads a column 1.17 ms: a level of
// shuffles costs the walk about as much as 25 rows a thread.)
constexpr int G = D % 16 == 0 ? 4 : D % 8 == 0 ? 2 : 1;
constexpr bool VEC = D % (4 * G) == 0;               // false: one thread a column, one value a load
constexpr int SL = D / G;                            // rows of a column per thread
constexpr int CS = (D % 16 == 0 && D > 16) ? 16 : D;  // columns of S per CTA
constexpr int NS = D / CS;                           // CTAs per head
constexpr int NT = ((CS * G + 31) / 32) * 32;
constexpr int CH = 16;                               // tokens per chunk
static_assert(D >= 4 && D <= 256, "head size of the delta rule kernel: 4 to 256");

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// What the walk reads per token and head is one record, prepared by a kernel that is parallel over
// tokens and copied to shared memory as it is:
//   u, r * w, w, a * u, k   five vectors over the rows of S
//   v                       D values
//   alpha, beta             alpha = r . (a * u), beta = r . k
// With them the output needs only the OLD state:
//   o_j = sum_i r_i S'_ij = (r * w) . S_j  -  alpha (u . S_j)  +  beta v_j
// so a token costs two independent sums over a column of S and one update, of which only one multiply-add
// waits for the sums.  Records of one head lie token after token in global memory: a chunk is one
// contiguous block.  (Loads into registers instead, issued before the walk of the chunk before, held the
// walk's own shared-memory loads back behind them in the load pipe.)
constexpr int PV = 5;
// A vector over the rows of S lies row block by row block: thread g's rows g * SL .. g * SL + SL - 1
// together, then four floats of padding, so that a thread's share is consecutive 16-byte loads and the G
// threads of a column hit different banks.
constexpr int SLP = VEC ? SL + 4 : SL;
constexpr int RL = G * SLP;
constexpr int REC = (PV * RL + D + 2 + 3) / 4 * 4;      // floats of a record
constexpr int OFF_V = PV * RL, OFF_AB = PV * RL + D;
__device__ __forceinline__ int at_row(int i) { return (i / SL) * SLP + (i % SL); }
// row of S that thread g holds in register ii
__device__ __forceinline__ int row_of(int g, int ii) { return g * SL + ii; }

struct DeltaParams {
  float* out;           // [tokens, heads * D]: each head's raw output o = S^T r
  const float* rec;     // [heads][tokens][REC]
  int tokens;
  float* state;         // [slots, heads, D, D] floats
  const int* q_start;   // [requests + 1]
  const int* state_slot;
  int heads, n_slots, write;
};

struct DeltaShared {
  float rec[2][CH][REC];
};

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// A thread's SL values of one vector of D values in shared memory.
__device__ __forceinline__ void load_rows(float (&dst)[SL], const float* vec, int g) {
  if constexpr (VEC) {
#pragma unroll
    for (int q = 0; q < SL / 4; ++q) {
      const float4 t = reinterpret_cast<const float4*>(vec + g * SLP)[q];
      dst[4 * q] = t.x, dst[4 * q + 1] = t.y, dst[4 * q + 2] = t.z, dst[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int ii = 0; ii < SL; ++ii) dst[ii] = vec[g * SLP + ii];
  }
}

template <typename T>
__global__ void __launch_bounds__(NT) delta_rule_kernel(DeltaParams p) {
  extern __shared__ __align__(16) uint8_t delta_smem[];
  static_assert(REC % 4 == 0 && (!VEC || (SLP % 4 == 0 && RL % 4 == 0)), "16-byte loads");
  DeltaShared& sh = *reinterpret_cast<DeltaShared*>(delta_smem);
  pdl_trigger();
  pdl_wait();
  const int h = blockIdx.x, req = blockIdx.y;
  const int tid = threadIdx.x;
  const int j = blockIdx.z * CS + tid / G, g = tid % G;      // this thread's column of S and its rows' block
  const bool live = tid / G < CS;
  const int row0 = p.q_start[req], row1 = p.q_start[req + 1];
  const int slot = p.state_slot[req];
  if (slot == -1) {      // a request of padding (length zero in a padded batch): zeros out, no state
    const int jj = blockIdx.z * CS + tid / G;
    if (tid / G < CS && tid % G == 0)
      for (int t = row0; t < row1; ++t) p.out[(size_t)t * p.heads * D + h * D + jj] = 0.f;
    return;
  }
  if (slot < 0 || slot >= p.n_slots) {
    if (tid == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  float* S_g = p.state + ((size_t)slot * p.heads + h) * D * D;
  float S[SL];
#pragma unroll
  for (int ii = 0; ii < SL; ++ii) S[ii] = live ? S_g[(size_t)row_of(g, ii) * D + j] : 0.f;
  const int ld_out = p.heads * D;
  const float* records = p.rec + (size_t)h * p.tokens * REC;

  // chunk c of the request -> buffer c & 1, sixteen bytes a copy
  auto fetch = [&](int t0, int buf) {
    const int n16 = min(CH, row1 - t0) * (REC / 4);
    const float* src = records + (size_t)t0 * REC;
    const uint32_t dst = smem_u32(&sh.rec[buf][0][0]);
    for (int c = tid; c < n16; c += NT) cp_async_16(dst + 16 * c, src + 4 * c);
    cp_async_commit_group();
  };

  fetch(row0, 0);
  int buf = 0;
  for (int t0 = row0; t0 < row1; t0 += CH, buf ^= 1) {
    const int n = min(CH, row1 - t0);
    cp_async_wait_all();
    __syncthreads();       // the chunk has landed for everyone, and the other buffer's readers are done
    if (t0 + CH < row1) fetch(t0 + CH, buf ^ 1);
    // ---- the recurrence, token by token ---------------------------------------------------
    for (int tok = 0; tok < n; ++tok) {
      // All of the token's values are asked for at once; what does not wait for the sums over the column
      // (w * S + k * v_j) is formed beside them, so that one multiply-add follows the shuffles.
      float u[SL], rw_[SL], w[SL], au[SL], kk[SL];
      const float* rec = sh.rec[buf][tok];
      load_rows(u, rec, g);
      load_rows(rw_, rec + RL, g);
      load_rows(w, rec + 2 * RL, g);
      load_rows(au, rec + 3 * RL, g);
      load_rows(kk, rec + 4 * RL, g);
      const float vj = live ? rec[OFF_V + j] : 0.f;
      const float alpha = rec[OFF_AB], beta = rec[OFF_AB + 1];
      float sa0 = 0.f, sa1 = 0.f, rw0 = 0.f, rw1 = 0.f;
#pragma unroll
      for (int ii = 0; ii < SL; ii += 2) {
        sa0 = fmaf(u[ii], S[ii], sa0);
        rw0 = fmaf(rw_[ii], S[ii], rw0);
        if (ii + 1 < SL) {
          sa1 = fmaf(u[ii + 1], S[ii + 1], sa1);
          rw1 = fmaf(rw_[ii + 1], S[ii + 1], rw1);
        }
      }
      float sa = sa0 + sa1, rw = rw0 + rw1;
#pragma unroll
      for (int ii = 0; ii < SL; ++ii) S[ii] = fmaf(kk[ii], vj, w[ii] * S[ii]);
#pragma unroll
      for (int o = 1; o < G; o <<= 1) {
        sa += __shfl_xor_sync(0xffffffffu, sa, o);
        rw += __shfl_xor_sync(0xffffffffu, rw, o);
      }
#pragma unroll
      for (int ii = 0; ii < SL; ++ii) S[ii] = fmaf(-au[ii], sa, S[ii]);
      if (live && g == 0) p.out[(size_t)(t0 + tok) * ld_out + h * D + j] = fmaf(beta, vj, fmaf(-alpha, sa, rw));
    }
  }
  if (p.write && live) {
#pragma unroll
    for (int ii = 0; ii < SL; ++ii) S_g[(size_t)row_of(g, ii) * D + j] = S[ii];
  }
}

// Per token and head, everything of the recurrence that does not depend on the state, in 32-bit:
// decay w = exp(-rate * sigmoid(d + bias)), removal a = sigmoid(. + bias), unit key u, and the products
// the walk uses.  One CTA per token, a warp per head at a time.
template <typename T>
__global__ void __launch_bounds__(256) delta_prepare_kernel(float* __restrict__ records, int tokens,
                                                            const float* __restrict__ r, const float* __restrict__ k,
                                                            const float* __restrict__ v, const float* __restrict__ a,
                                                            int ld, const float* __restrict__ d, int ld_d,
                                                            const T* __restrict__ d_bias, const T* __restrict__ a_bias,
                                                            int heads, float decay_rate) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int h = blockIdx.y * 8 + warp; h < heads; h += 8 * gridDim.y) {
    const size_t at = (size_t)t * ld + h * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss += k[at + i] * k[at + i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + 1e-6f);
    float* dst = records + ((size_t)h * tokens + t) * REC;
    float al = 0.f, be = 0.f;
    for (int i = lane; i < D; i += 32) {
      const float kk = k[at + i], rr = r[at + i];
      const float w = expf(-decay_rate * sigmoidf_(d[(size_t)t * ld_d + h * D + i] + to_f32(d_bias[h * D + i])));
      const float u = kk * inv, au = sigmoidf_(a[at + i] + to_f32(a_bias[h * D + i])) * u;
      const int ir = at_row(i);
      dst[ir] = u, dst[RL + ir] = rr * w, dst[2 * RL + ir] = w, dst[3 * RL + ir] = au, dst[4 * RL + ir] = kk;
      dst[OFF_V + i] = v[at + i];
      al = fmaf(rr, au, al);
      be = fmaf(rr, kk, be);
    }
    al = warp_sum(al);
    be = warp_sum(be);
    if (lane == 0) dst[OFF_AB] = al, dst[OFF_AB + 1] = be;
  }
}

// Each head's raw output divided by its root mean square, times a plain weight and sigmoid(gate),
// rounded to T: one CTA per token, a warp per head at a time.
template <typename T>
__global__ void __launch_bounds__(256) delta_finish_kernel(T* __restrict__ out, const float* __restrict__ raw,
                                                           const float* __restrict__ gate, int ld_gate,
                                                           const T* __restrict__ norm_w, int heads, float eps) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int h = blockIdx.y * 8 + warp; h < heads; h += 8 * gridDim.y) {
    const float* o = raw + ((size_t)t * heads + h) * D;
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) ss += o[i] * o[i];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)D + eps);
    for (int i = lane; i < D; i += 32)
      out[((size_t)t * heads + h) * D + i] =
          from_f32<T>(o[i] * inv * to_f32(norm_w[h * D + i]) * sigmoidf_(gate[(size_t)t * ld_gate + h * D + i]));
  }
}

// out (T) [tokens, n] = tanh(x [tokens, ld]) for the low-rank middle of the decay's projection
template <typename T>
__global__ void __launch_bounds__(256) tanh_cast_kernel(T* __restrict__ out, const float* __restrict__ x, long long tokens,
                                                        int n, int ld) {
  pdl_trigger();
  pdl_wait();
  const long long total = tokens * n;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < total; i += (long long)gridDim.x * 256)
    out[i] = from_f32<T>(tanhf(x[(i / n) * ld + (i % n)]));
}

}  // namespace

LAB_EXPORT int lab_delta_rule_head_dim() { return D; }

// scratch: floats for the heads' raw outputs and the records
LAB_EXPORT long long lab_delta_rule_scratch(int tokens, int heads) {
  return (long long)tokens * heads * (D + REC) + REC;
}

LAB_EXPORT int lab_delta_rule(void* out, float* scratch, const float* r, const float* k, const float* v,
                              const float* g, const float* a, int ld, const float* d, int ld_d, const void* d_bias,
                              const void* a_bias, const void* norm_w, float* state, const int* q_start,
                              const int* state_slot, int tokens, int n_requests, int heads, int n_slots, int write,
                              float eps, float decay_rate, int dtype, cudaStream_t stream) {
  if (n_requests <= 0 || heads <= 0 || tokens <= 0) return 0;
  float* raw = scratch;
  float* records = raw + (size_t)tokens * heads * D;      // tokens * heads * D is a multiple of 4 floats or not:
  records += (4 - ((size_t)tokens * heads * D) % 4) % 4;  // records start on 16 bytes (one spare record is asked for)
  DeltaParams p;
  p.out = raw; p.rec = records; p.tokens = tokens; p.state = state; p.q_start = q_start;
  p.state_slot = state_slot; p.heads = heads; p.n_slots = n_slots; p.write = write;
  const size_t smem = sizeof(DeltaShared);
  const dim3 grid(heads, n_requests, NS);
  // the two kernels that are parallel over tokens: a warp per (token, head); with few tokens the heads
  // spread over CTAs as well
  const dim3 per_token(tokens, tokens >= 512 ? 1 : (heads + 7) / 8);
  cudaError_t e;
  if (dtype == LAB_F32) {
    e = cudaFuncSetAttribute(delta_rule_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lab_launch(delta_prepare_kernel<float>, per_token, dim3(256), 0, stream, records, tokens, r, k, v, a, ld, d,
               ld_d, (const float*)d_bias, (const float*)a_bias, heads, decay_rate);
    lab_launch(delta_rule_kernel<float>, grid, dim3(NT), smem, stream, p);
    lab_launch(delta_finish_kernel<float>, per_token, dim3(256), 0, stream, (float*)out, (const float*)raw, g, ld,
               (const float*)norm_w, heads, eps);
  } else {
    e = cudaFuncSetAttribute(delta_rule_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    lab_launch(delta_prepare_kernel<__nv_bfloat16>, per_token, dim3(256), 0, stream, records, tokens, r, k, v, a,
               ld, d, ld_d, (const __nv_bfloat16*)d_bias, (const __nv_bfloat16*)a_bias, heads, decay_rate);
    lab_launch(delta_rule_kernel<__nv_bfloat16>, grid, dim3(NT), smem, stream, p);
    lab_launch(delta_finish_kernel<__nv_bfloat16>, per_token, dim3(256), 0, stream, (__nv_bfloat16*)out,
               (const float*)raw, g, ld, (const __nv_bfloat16*)norm_w, heads, eps);
  }
  LAB_LAUNCH_CHECK();
}

LAB_EXPORT int lab_tanh_cast(void* out, const float* x, long long tokens, int n, int ld, int dtype,
                             cudaStream_t stream) {
  const long long total = tokens * n;
  if (total <= 0) return 0;
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (dtype == LAB_F32)
    lab_launch(tanh_cast_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)out, x, tokens, n, ld);
  else
    lab_launch(tanh_cast_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, (__nv_bfloat16*)out, x, tokens, n,
               ld);
  LAB_LAUNCH_CHECK();
}
