// Recurrent mixers whose state per head is a matrix S [key channel, value channel] with a scalar decay:
//
//     S_t = a_t * S_{t-1} + (s_t * k_t) v_t^T,        o_t = S_t^T q_t
//
// a_t is a constant of the head (linear attention with a fixed decay) or a number per token and head (a
// state-space mixer, where a_t = exp(-exp(A_log) * dt_t) and s_t = dt_t); q and k may be shared by the
// heads of a group.  The state is 32-bit, is read at a request's first row of the step and written back
// after its last, and every product and sum of the recurrence is 32-bit, token by token in order, so a
// position's result does not depend on how the sequence was cut into steps.
//
//   decay_scan        the recurrence over each request's rows (any number of rows, single tokens included)
//   ssm_prepare       for a state-space mixer, from the 32-bit input projection [z | x | B | C | dt]: the
//                     causal convolution per channel of x, B, C over the last `taps` inputs (the inputs
//                     before a step's first row come from the request's kept inputs) with bias and SiLU;
//                     dt = softplus(dt + dt_bias); a = exp(-exp(A_log) * dt)
//   ssm_keep_inputs   the request's last taps - 1 inputs of x, B, C replace the kept ones
//   gated_norm        the heads' outputs side by side (+ skip * x), a gate, an RMS norm in equal parts with
//                     a weight, in either order (gate first with SiLU, or norm first with a sigmoid),
//                     rounded to T for the output projection
//
// T says how weights are stored and how the last result is rounded.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int SCAN_P = 4;     // threads that share one column of the state
constexpr int SCAN_CT = 16;   // tokens staged per chunk

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
// SiLU by the hardware's 2^x and reciprocal approximations (relative error about 2^-21, as the attention
// kernels' softmax has it): a few instructions instead of the seventy of the exact exponential and division,
// which the recurrence's helpers would otherwise spend longer on than its walkers on their chunk.
__device__ __forceinline__ float silu_quick(float z) { return __fdividef(z, 1.0f + fast_exp2(-1.4426950408889634f * z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct ScanParams {
  float* out;            // [tokens, ld_o]: head h at h * V
  int ld_o;
  const float* q;        // [tokens, ld_qk]: group g at g * N
  const float* k;
  int ld_qk;
  const float* v;        // [tokens, ld_v]: head h at h * V
  int ld_v;
  const float* a_tok;    // [tokens, ld_a] decay per token and head, or null
  const float* s_tok;    // [tokens, ld_a] scale of the key per token and head, or null (1)
  int ld_a;
  const float* a_head;   // [H] decay per head, read when a_tok is null
  float* state;          // [slots, H, N, V]
  const int* q_start;
  const int* state_slot;
  int n_slots, H, G, N, V, act, write;
  int vec;               // q, k, v rows may be copied 16 bytes at a time
};

// grid (slices of V, heads, requests); block 2 * SCAN_P * Vs threads in two halves.
//
// Walkers (the first SCAN_P * Vs threads): thread (j, part) keeps rows part * R .. part * R + R - 1 of column
// slice * Vs + j of the state in registers (R a multiple of 4: the rows' keys and queries come from shared
// memory four at a time; the four threads' shares of a token's keys lie R + 4 floats apart, which spreads
// their 16-byte loads over the banks).  A token costs a walker 2 R multiply-adds behind R / 2 loads; the four
// walkers of a column add their shares of the output by two shuffles.  The next token's keys, queries and
// value are loaded before the current token's arithmetic (up to R = 16; beyond, registers do not allow it).
// The walk is one dependent chain per request and head: its time is the number of tokens times that step,
// whatever the number of CTAs, so nothing else may sit on it.
//
// Helpers (the other half) keep everything else off that chain: while the walkers are on chunk c (16 tokens),
// the helpers apply the SiLU to chunk c + 1, whose rows their cp.async copies have brought (16 bytes a copy
// where the operands' addresses allow it: `vec`), and start the copies of chunk c + 2 into the buffer the
// walkers left one chunk ago.  Three buffers, one barrier of the whole CTA per chunk.
template <int R>
__global__ void __launch_bounds__(256) decay_scan_kernel(ScanParams p) {
  extern __shared__ __align__(16) float smem[];
  constexpr int RS = R + 4;                      // floats between two threads' shares of a token's keys
  constexpr int NP = SCAN_P * RS;                // floats of a token's keys (or queries) in shared memory
  constexpr bool AHEAD = R <= 16;                // the next token's operands are loaded a token ahead
  pdl_trigger();
  const int walkers = blockDim.x / 2, Vs = walkers / SCAN_P;
  const int tok_floats = 2 * NP + Vs + 4;        // k | q | v | a | s | (two unused, which keep rows 16-byte aligned)
  const int h = blockIdx.y, r = blockIdx.z, g = h / (p.H / p.G);
  const bool helper = threadIdx.x >= walkers;
  const int tid = helper ? threadIdx.x - walkers : threadIdx.x;      // index within the half
  const int j = tid / SCAN_P, part = tid % SCAN_P;
  const int col0 = blockIdx.x * Vs, col = col0 + j;
  const int t0 = p.q_start[r], n_tok = p.q_start[r + 1] - t0;
  const int slot = p.state_slot[r];
  if (n_tok <= 0 || slot == -1) {      // nothing to do, or rows of padding (their output is never read)
    pdl_wait();
    return;
  }
  if (slot < 0 || slot >= p.n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    pdl_wait();
    return;
  }
  // padding of the key channels and of the columns stays zero for the whole walk: the copies never touch it
  for (int i = threadIdx.x; i < 3 * SCAN_CT * tok_floats; i += blockDim.x) smem[i] = 0.f;
  __syncthreads();
  pdl_wait();

  const int n_chunks = (n_tok + SCAN_CT - 1) / SCAN_CT;
  const int v_cols = min(Vs, p.V - col0);
  auto buffer = [&](int chunk) { return smem + (chunk % 3) * SCAN_CT * tok_floats; };

  // ---- helpers' pieces ----
  auto at = [](int n) { return (n / R) * RS + (n % R); };      // where key channel n lies within a token's keys
  // One loop over all of a chunk's copies (tokens x pieces), so that every helper has a few copies in flight
  // instead of the helpers walking the tokens one after the other.
  auto issue = [&](int chunk) {
    const int first = chunk * SCAN_CT, cnt = min(SCAN_CT, n_tok - first);
    float* base = buffer(chunk);
    const float* k0 = p.k + (size_t)(t0 + first) * p.ld_qk + g * p.N;
    const float* q0 = p.q + (size_t)(t0 + first) * p.ld_qk + g * p.N;
    const float* v0 = p.v + (size_t)(t0 + first) * p.ld_v + h * p.V + col0;
    if (p.vec) {
      const int nk = p.N / 4, nv = v_cols / 4, per = 2 * nk + nv;
      for (int e = tid; e < cnt * per; e += walkers) {
        const int tt = e / per, c = e - tt * per;
        float* dst = base + tt * tok_floats;
        if (c < nk) cp_async16(dst + at(4 * c), k0 + (size_t)tt * p.ld_qk + 4 * c);
        else if (c < 2 * nk) cp_async16(dst + NP + at(4 * (c - nk)), q0 + (size_t)tt * p.ld_qk + 4 * (c - nk));
        else cp_async16(dst + 2 * NP + 4 * (c - 2 * nk), v0 + (size_t)tt * p.ld_v + 4 * (c - 2 * nk));
      }
    } else {
      const int per = 2 * p.N + v_cols;
      for (int e = tid; e < cnt * per; e += walkers) {
        const int tt = e / per, c = e - tt * per;
        float* dst = base + tt * tok_floats;
        if (c < p.N) cp_async4(dst + at(c), k0 + (size_t)tt * p.ld_qk + c);
        else if (c < 2 * p.N) cp_async4(dst + NP + at(c - p.N), q0 + (size_t)tt * p.ld_qk + (c - p.N));
        else cp_async4(dst + 2 * NP + (c - 2 * p.N), v0 + (size_t)tt * p.ld_v + (c - 2 * p.N));
      }
    }
    if (p.a_tok != nullptr && tid < 2 * cnt) {      // a token's decay and key scale: one helper each
      const int tt = tid >> 1, which = tid & 1;
      const float* src = which == 0 ? p.a_tok : p.s_tok;
      if (src != nullptr)
        cp_async4(base + tt * tok_floats + 2 * NP + Vs + which, src + (size_t)(t0 + first + tt) * p.ld_a + h);
    }
  };
  // after the copies of `chunk` have landed for every helper: SiLU of q, k and v, once per element
  auto finish = [&](int chunk) {
    asm volatile("bar.sync 1, %0;" ::"r"(walkers) : "memory");      // the helpers alone
    if (!p.act) return;
    const int cnt = min(SCAN_CT, n_tok - chunk * SCAN_CT), per = (2 * NP + Vs) / 4;
    float* base = buffer(chunk);
    for (int e = tid; e < cnt * per; e += walkers) {
      const int tt = e / per, c = e - tt * per;
      float4* at4 = reinterpret_cast<float4*>(base + tt * tok_floats) + c;
      float4 z = *at4;
      z.x = silu_quick(z.x), z.y = silu_quick(z.y), z.z = silu_quick(z.z), z.w = silu_quick(z.w);
      *at4 = z;
    }
  };

  float S[R];
  float* st = p.state + ((size_t)slot * p.H + h) * p.N * p.V;
  float a_const = 0.f;
  if (helper) {
    issue(0);
    cp_async_commit_group();
    if (n_chunks > 1) issue(1);
    cp_async_commit_group();
    cp_async_wait_group<1>();
    finish(0);
  } else {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int n = part * R + i;
      S[i] = (n < p.N && col < p.V) ? st[(size_t)n * p.V + col] : 0.f;
    }
    if (p.a_tok == nullptr) a_const = p.a_head[h];
  }
  __syncthreads();

  for (int c = 0; c < n_chunks; ++c) {
    if (helper) {
      if (c + 2 < n_chunks) issue(c + 2);      // into the buffer the walkers left at the last barrier
      cp_async_commit_group();
      if (c + 1 < n_chunks) {
        cp_async_wait_group<1>();              // all but the copies just started: chunk c + 1 is here
        finish(c + 1);
      }
    } else {
      const int cnt = min(SCAN_CT, n_tok - c * SCAN_CT);
      const float* base = buffer(c);
      float* out = p.out + (size_t)(t0 + c * SCAN_CT) * p.ld_o + h * p.V + col;
      float4 kk[R / 4], qq[R / 4];
      float a, vj;
      auto load = [&](int tt, float4* k_to, float4* q_to, float& a_to, float& v_to) {
        const float* tok = base + tt * tok_floats;
        const float4* k4 = reinterpret_cast<const float4*>(tok + part * RS);
        const float4* q4 = reinterpret_cast<const float4*>(tok + NP + part * RS);
#pragma unroll
        for (int i = 0; i < R / 4; ++i) k_to[i] = k4[i], q_to[i] = q4[i];
        a_to = p.a_tok != nullptr ? tok[2 * NP + Vs] : a_const;
        v_to = tok[2 * NP + j];
        if (p.s_tok != nullptr) v_to *= tok[2 * NP + Vs + 1];
      };
      if (AHEAD) load(0, kk, qq, a, vj);
      for (int tt = 0; tt < cnt; ++tt) {
        float4 kn[AHEAD ? R / 4 : 1], qn[AHEAD ? R / 4 : 1];
        float an = 0.f, vn = 0.f;
        if (AHEAD) {
          if (tt + 1 < cnt) load(tt + 1, kn, qn, an, vn);
        } else {
          load(tt, kk, qq, a, vj);
        }
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < R / 4; ++i) {
          S[4 * i + 0] = fmaf(a, S[4 * i + 0], kk[i].x * vj);
          S[4 * i + 1] = fmaf(a, S[4 * i + 1], kk[i].y * vj);
          S[4 * i + 2] = fmaf(a, S[4 * i + 2], kk[i].z * vj);
          S[4 * i + 3] = fmaf(a, S[4 * i + 3], kk[i].w * vj);
          acc[0] = fmaf(S[4 * i + 0], qq[i].x, acc[0]);
          acc[1] = fmaf(S[4 * i + 1], qq[i].y, acc[1]);
          acc[2] = fmaf(S[4 * i + 2], qq[i].z, acc[2]);
          acc[3] = fmaf(S[4 * i + 3], qq[i].w, acc[3]);
        }
        float total = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        total += __shfl_xor_sync(0xffffffffu, total, 1);
        total += __shfl_xor_sync(0xffffffffu, total, 2);
        if (part == 0 && col < p.V) out[(size_t)tt * p.ld_o] = total;
        if (AHEAD) {
#pragma unroll
          for (int i = 0; i < R / 4; ++i) kk[i] = kn[i], qq[i] = qn[i];
          a = an, vj = vn;
        }
      }
    }
    __syncthreads();
  }
  if (helper) {
    cp_async_wait_group<0>();
  } else if (p.write) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int n = part * R + i;
      if (n < p.N && col < p.V) st[(size_t)n * p.V + col] = S[i];
    }
  }
}

// ---- state-space mixer: convolution, step sizes, decays ---------------------------------------
struct SsmParams {
  const float* proj;     // [tokens, ld]
  int ld, conv_at, dt_at, channels, taps, H;
  float* kept;           // [slots, taps - 1, channels]: the request's last inputs, oldest first
  const int* row_req;
  const int* q_start;
  const int* state_slot;
  int n_slots;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) ssm_prepare_kernel(float* __restrict__ conv_out, float* __restrict__ dt_out,
                                                               float* __restrict__ a_out, const T* __restrict__ taps_w,
                                                               const T* __restrict__ taps_b, const T* __restrict__ dt_bias,
                                                               const T* __restrict__ a_log, SsmParams p) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, r = p.row_req[t], first = p.q_start[r], slot = p.state_slot[r];
  const int K = p.taps, C = p.channels;
  // grid (rows, blocks of channels): a thread forms one channel, so that a row's loads are all in flight at
  // once (a step of few rows is bound by their latency); the first block of a row also forms its step sizes
  const int c = blockIdx.y * kThreads + threadIdx.x;
  const bool heads_too = blockIdx.y == 0;
  if (slot == -1) {       // a row of padding
    if (c < C) conv_out[(size_t)t * C + c] = 0.f;
    for (int h = threadIdx.x; heads_too && h < p.H; h += kThreads) dt_out[(size_t)t * p.H + h] = a_out[(size_t)t * p.H + h] = 0.f;
    return;
  }
  if (slot < 0 || slot >= p.n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const float* kept = p.kept + (size_t)slot * (K - 1) * C;
  if (c < C) {
    float acc = to_f32(taps_b[c]);
    for (int jj = 0; jj < K; ++jj) {
      const int src = t - (K - 1) + jj;       // the last tap meets the row itself
      const float u = src >= first ? p.proj[(size_t)src * p.ld + p.conv_at + c]
                                   : kept[(size_t)((K - 1) + (src - first)) * C + c];
      acc = fmaf(to_f32(taps_w[(size_t)c * K + jj]), u, acc);
    }
    conv_out[(size_t)t * C + c] = silu_f(acc);
  }
  for (int h = threadIdx.x; heads_too && h < p.H; h += kThreads) {
    const float dt = softplus_f(p.proj[(size_t)t * p.ld + p.dt_at + h] + to_f32(dt_bias[h]));
    dt_out[(size_t)t * p.H + h] = dt;
    a_out[(size_t)t * p.H + h] = expf(-expf(to_f32(a_log[h])) * dt);
  }
}

// grid (requests, blocks of channels), after every row of the step has read the kept inputs.  A thread walks
// the kept rows of its one channel oldest first: what it overwrites it has already moved.
__global__ void __launch_bounds__(kThreads) ssm_keep_inputs_kernel(SsmParams p, int requests) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.x;
  const int first = p.q_start[r], n = p.q_start[r + 1] - first, slot = p.state_slot[r];
  if (n <= 0 || slot == -1) return;
  if (slot < 0 || slot >= p.n_slots) {
    if (threadIdx.x == 0) lab_set_error(LAB_ERR_PAGE_RANGE);
    return;
  }
  const int K1 = p.taps - 1, C = p.channels;
  float* kept = p.kept + (size_t)slot * K1 * C;
  const int c = blockIdx.y * kThreads + threadIdx.x;
  if (c >= C) return;
  for (int i = 0; i < K1; ++i) {
    const int s = n - K1 + i;               // the step's row that becomes kept row i
    kept[(size_t)i * C + c] = s >= 0 ? p.proj[(size_t)(first + s) * p.ld + p.conv_at + c] : kept[(size_t)(i + n) * C + c];
  }
}

// ---- gate and norm of the heads' outputs ------------------------------------------------------
// y[i] = o[t, i] + skip[head of i] * x[t, i]; gate_first: y *= silu(gate), then y / rms(part of i) * w;
// else y / rms(part) * w * sigmoid(gate); times `mult`, rounded to T.
template <typename T>
__global__ void __launch_bounds__(kThreads) gated_norm_kernel(T* __restrict__ out, int ld_out, const float* __restrict__ o,
                                                              int ld_o, const float* __restrict__ x, int ld_x,
                                                              const T* __restrict__ skip, int head_size,
                                                              const float* __restrict__ gate, int ld_g,
                                                              const T* __restrict__ w, int width, int parts,
                                                              int gate_first, float eps, float mult) {
  extern __shared__ float row[];      // [width]
  __shared__ float scratch[32];
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int part_size = width / parts;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    float y = o[(size_t)t * ld_o + i];
    if (skip != nullptr) y = fmaf(to_f32(skip[i / head_size]), x[(size_t)t * ld_x + i], y);
    if (gate_first) y *= silu_f(gate[(size_t)t * ld_g + i]);
    row[i] = y;
  }
  __syncthreads();
  for (int g = 0; g < parts; ++g) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < part_size; i += kThreads) {
      const float y = row[g * part_size + i];
      ss += y * y;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)part_size + eps);
    for (int i = threadIdx.x; i < part_size; i += kThreads) {
      const int c = g * part_size + i;
      float y = row[c] * inv * to_f32(w[c]);
      if (!gate_first) y *= sigmoid_f(gate[(size_t)t * ld_g + c]);
      out[(size_t)t * ld_out + c] = from_f32<T>(y * mult);
    }
  }
}

template <int R>
int launch_scan(const ScanParams& p, int requests, int vs, cudaStream_t stream) {
  const size_t smem = (size_t)3 * SCAN_CT * (2 * SCAN_P * (R + 4) + vs + 4) * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(decay_scan_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid((p.V + vs - 1) / vs, p.H, requests);
  return (int)lab_launch(decay_scan_kernel<R>, grid, dim3(2 * SCAN_P * vs), smem, stream, p);
}

}  // namespace

// Largest key size the recurrence kernel is built for.
LAB_EXPORT int lab_decay_scan_max_keys() { return SCAN_P * 64; }

// vs: columns of the state a CTA takes (8, 16 or 32).
LAB_EXPORT int lab_decay_scan(float* out, int ld_o, const float* q, const float* k, int ld_qk, const float* v, int ld_v,
                              const float* a_tok, const float* s_tok, int ld_a, const float* a_head, float* state,
                              const int* q_start, const int* state_slot, int requests, int n_slots, int H, int G, int N,
                              int V, int act, int write, int vs, cudaStream_t stream) {
  if (requests <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || N <= 0 || V <= 0 || (vs != 8 && vs != 16 && vs != 32)) return (int)cudaErrorInvalidValue;
  if (a_tok == nullptr && a_head == nullptr) return (int)cudaErrorInvalidValue;
  ScanParams p;
  p.out = out; p.ld_o = ld_o; p.q = q; p.k = k; p.ld_qk = ld_qk; p.v = v; p.ld_v = ld_v; p.a_tok = a_tok;
  p.s_tok = s_tok; p.ld_a = ld_a; p.a_head = a_head; p.state = state; p.q_start = q_start; p.state_slot = state_slot;
  p.n_slots = n_slots; p.H = H; p.G = G; p.N = N; p.V = V; p.act = act; p.write = write;
  // 16-byte copies: every row of q, k and v, and every head's and slice's start in it, on a 16-byte boundary
  p.vec = N % 4 == 0 && V % 4 == 0 && ld_qk % 4 == 0 && ld_v % 4 == 0 &&
          ((((uintptr_t)q) | ((uintptr_t)k) | ((uintptr_t)v)) & 15) == 0;
  if (N <= SCAN_P * 4) return launch_scan<4>(p, requests, vs, stream);
  if (N <= SCAN_P * 8) return launch_scan<8>(p, requests, vs, stream);
  if (N <= SCAN_P * 16) return launch_scan<16>(p, requests, vs, stream);
  if (N <= SCAN_P * 32) return launch_scan<32>(p, requests, vs, stream);
  if (N <= SCAN_P * 64) return launch_scan<64>(p, requests, vs, stream);
  return (int)cudaErrorInvalidValue;
}

LAB_EXPORT int lab_ssm_prepare(float* conv_out, float* dt_out, float* a_out, const float* proj, int ld, int conv_at,
                               int dt_at, int channels, int taps, int H, const void* taps_w, const void* taps_b,
                               const void* dt_bias, const void* a_log, float* kept, const int* row_req,
                               const int* q_start, const int* state_slot, int tokens, int requests, int n_slots,
                               int write, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (taps < 1 || channels <= 0 || H <= 0) return (int)cudaErrorInvalidValue;
  SsmParams p;
  p.proj = proj; p.ld = ld; p.conv_at = conv_at; p.dt_at = dt_at; p.channels = channels; p.taps = taps; p.H = H;
  p.kept = kept; p.row_req = row_req; p.q_start = q_start; p.state_slot = state_slot; p.n_slots = n_slots;
  const int c_blocks = (channels + kThreads - 1) / kThreads;
  if (c_blocks > 65535) return (int)cudaErrorInvalidValue;
  cudaError_t e;
  if (dtype == LAB_F32)
    e = lab_launch(ssm_prepare_kernel<float>, dim3(tokens, c_blocks), dim3(kThreads), 0, stream, conv_out, dt_out, a_out,
                   (const float*)taps_w, (const float*)taps_b, (const float*)dt_bias, (const float*)a_log, p);
  else
    e = lab_launch(ssm_prepare_kernel<__nv_bfloat16>, dim3(tokens, c_blocks), dim3(kThreads), 0, stream, conv_out, dt_out, a_out,
                   (const __nv_bfloat16*)taps_w, (const __nv_bfloat16*)taps_b, (const __nv_bfloat16*)dt_bias,
                   (const __nv_bfloat16*)a_log, p);
  if (e != cudaSuccess) return (int)e;
  if (write && taps > 1)
    return (int)lab_launch(ssm_keep_inputs_kernel, dim3(requests, c_blocks), dim3(kThreads), 0, stream, p, requests);
  return 0;
}

LAB_EXPORT int lab_gated_norm(void* out, int ld_out, const float* o, int ld_o, const float* x, int ld_x, const void* skip,
                              int head_size, const float* gate, int ld_g, const void* w, int tokens, int width, int parts,
                              int gate_first, float eps, float mult, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (parts <= 0 || width % parts) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)width * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == LAB_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(gated_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lab_launch(gated_norm_kernel<float>, dim3(tokens), dim3(kThreads), smem, stream, (float*)out, ld_out, o, ld_o, x, ld_x,
               (const float*)skip, head_size, gate, ld_g, (const float*)w, width, parts, gate_first, eps, mult);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(gated_norm_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    lab_launch(gated_norm_kernel<__nv_bfloat16>, dim3(tokens), dim3(kThreads), smem, stream, (__nv_bfloat16*)out, ld_out, o,
               ld_o, x, ld_x, (const __nv_bfloat16*)skip, head_size, gate, ld_g, (const __nv_bfloat16*)w, width, parts,
               gate_first, eps, mult);
  }
  LAB_LAUNCH_CHECK();
}
