// A recurrent block with a real-gated linear recurrence over channels (one number of state a
// channel), behind a short causal convolution:
//
//   x_t = projected x + bias                     [C]
//   u_t = conv bias + sum_j taps[:, K - 1 - j] x_(t - j)      (zeros ahead of a request's start)
//   r_t = sigmoid(zr_t + br), i_t = sigmoid(zi_t + bi)        (zr, zi: block-diagonal maps of u_t, made
//                                                              between the first and the second kernel)
//   a_t = exp(-c r_t softplus(lam)),  S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t
//   out_t = S_t * gelu_tanh(projected y + bias)
//
// Everything from x on is float32. Three kernels:
//
//   conv     per (token, channel): u from this step's rows and, for the first K - 1 tokens of a
//            portion, from the request's state slot (its last K - 1 inputs); state untouched.
//   gates    per (token, channel): a_t and b_t = sqrt(1 - a_t^2) i_t u_t, with 1 - a^2 taken as
//            -expm1(2 log a) so that decays close to one keep their digits; and y_t.
//   scan     per (request, channel), W warps a block each with a segment of the portion's tokens:
//            every warp folds its segment to (product of a, value from zero), the segments' starts
//            follow from those in order, and every warp walks its segment again from its start and
//            writes S_t y_t. Then the block moves the convolution's state on (the last K - 1 inputs).
//            The cut into segments depends on the portion's length only through rounding: a segment's
//            start is S_before * (product of a) + (value from zero), the same recurrence regrouped.
//
//   step     a step in which every request brings one token (decoding) runs all of the above in one
//            kernel: a block per (request, block of the gates' maps) makes its channels' u, takes the two
//            maps' products with it from the float32 matrices (a thread an output, the additions in the
//            order of the inputs), and moves S and the convolution's state on.
#include "common.cuh"

#define RGLRU_MAX_TAPS 16
#define RGLRU_SCAN_WARPS 16

namespace {

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename T>
__global__ void rglru_conv_kernel(const T* __restrict__ proj, int stride, int x_col, const float* __restrict__ x_bias,
                                  const float* __restrict__ taps, const float* __restrict__ conv_bias, int C, int K,
                                  const float* __restrict__ conv_state, const int* __restrict__ cu_seqlens,
                                  const int* __restrict__ state_slots, int num_seqs, float* __restrict__ u) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  // The token's request: the last one whose tokens begin at or before t (requests without tokens in
  // this step share their begin with the next one and are passed over).
  int lo = 0, hi = num_seqs;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid;
    else hi = mid;
  }
  const int seq = lo;
  const int begin = cu_seqlens[seq];
  const float* state = conv_state + (size_t)state_slots[seq] * (K - 1) * C;  // [K - 1][C], oldest first
  const float xb = x_bias ? x_bias[c] : 0.f;
  float acc = conv_bias ? conv_bias[c] : 0.f;
  for (int j = 0; j < K; ++j) {
    const int src = t - j;
    float x;
    if (src >= begin) x = to_f32(proj[(size_t)src * stride + x_col + c]) + xb;
    else x = state[(size_t)(K - 1 - (begin - src)) * C + c];  // begin - src in 1 .. K - 1
    acc = fmaf(taps[(size_t)c * K + (K - 1 - j)], x, acc);
  }
  u[(size_t)t * C + c] = acc;
}

// z: [blocks, tokens, 2 * bw] (r's outputs, then i's) as the batched product leaves them.
template <typename T>
__global__ void rglru_gates_kernel(const float* __restrict__ u, const float* __restrict__ z, const float* __restrict__ r_bias,
                                   const float* __restrict__ i_bias, const float* __restrict__ lam, float c_decay,
                                   const T* __restrict__ proj, int stride, int y_col, const float* __restrict__ y_bias,
                                   int C, int bw, int tokens, float* __restrict__ a_out, float* __restrict__ b_out,
                                   float* __restrict__ y_out) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int block = c / bw, o = c % bw;
  const float* zrow = z + ((size_t)block * tokens + t) * 2 * bw;
  const float r = 1.f / (1.f + expf(-(zrow[o] + r_bias[c])));
  const float i = 1.f / (1.f + expf(-(zrow[bw + o] + i_bias[c])));
  const float l = lam[c];
  const float softplus = fmaxf(l, 0.f) + log1pf(expf(-fabsf(l)));
  const float log_a = -c_decay * r * softplus;
  const size_t at = (size_t)t * C + c;
  a_out[at] = expf(log_a);
  b_out[at] = sqrtf(-expm1f(2.f * log_a)) * i * u[at];
  y_out[at] = gelu_tanh_f(to_f32(proj[(size_t)t * stride + y_col + c]) + (y_bias ? y_bias[c] : 0.f));
}

// grid (ceil(C / 32), requests); block 32 x W: lane = channel, warp = segment of tokens.
template <typename T>
__global__ void __launch_bounds__(32 * RGLRU_SCAN_WARPS) rglru_scan_kernel(
    const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ y, int C, int K,
    float* __restrict__ S_state, float* __restrict__ conv_state, const T* __restrict__ proj, int stride, int x_col,
    const float* __restrict__ x_bias, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
    T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float fold_a[RGLRU_SCAN_WARPS][32], fold_b[RGLRU_SCAN_WARPS][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int c = blockIdx.x * 32 + lane, seq = blockIdx.y;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  if (end <= begin) return;
  const bool live = c < C;
  const int n = end - begin;
  const int per = (n + warps - 1) / warps;
  const int t0 = begin + min(n, warp * per), t1 = begin + min(n, (warp + 1) * per);
  const size_t slot = (size_t)state_slots[seq];
  float S = 0.f;
  if (warps > 1) {
    float A = 1.f, B = 0.f;
    if (live) {
#pragma unroll 4
      for (int t = t0; t < t1; ++t) {
        const float at = a[(size_t)t * C + c];
        B = fmaf(at, B, b[(size_t)t * C + c]);
        A *= at;
      }
    }
    fold_a[warp][lane] = A, fold_b[warp][lane] = B;
    __syncthreads();
  }
  if (live) {
    S = S_state[slot * C + c];
    for (int w = 0; w < warp; ++w) S = fmaf(fold_a[w][lane], S, fold_b[w][lane]);
#pragma unroll 4
    for (int t = t0; t < t1; ++t) {
      const size_t at = (size_t)t * C + c;
      S = fmaf(a[at], S, b[at]);
      out[at] = from_f32<T>(S * y[at]);
    }
    if (t1 == end && t0 < t1) S_state[slot * C + c] = S;
  }
  // The convolution's state: the request's last K - 1 inputs, oldest first. The warp that holds the
  // portion's last token moves it on (every thread a channel: it reads what it needs before it writes).
  if (live && K > 1 && t1 == end && t0 < t1) {
    float* state = conv_state + slot * (K - 1) * C + c;
    float keep[RGLRU_MAX_TAPS];
    const float xb = x_bias ? x_bias[c] : 0.f;
#pragma unroll
    for (int i = 0; i < RGLRU_MAX_TAPS; ++i) {
      if (i >= K - 1) break;
      const int pos = n - (K - 1) + i;  // among this portion's tokens; negative: from the old state
      keep[i] = pos >= 0 ? to_f32(proj[(size_t)(begin + pos) * stride + x_col + c]) + xb : state[(size_t)(i + n) * C];
    }
#pragma unroll
    for (int i = 0; i < RGLRU_MAX_TAPS; ++i) {
      if (i >= K - 1) break;
      state[(size_t)i * C] = keep[i];
    }
  }
}

// grid (blocks of the maps, requests); gates [blocks, bw (in), 2 bw (out: r's, then i's)].
template <typename T>
__global__ void __launch_bounds__(1024) rglru_step_kernel(
    const T* __restrict__ proj, int stride, int x_col, int y_col, const float* __restrict__ x_bias,
    const float* __restrict__ y_bias, const float* __restrict__ taps, const float* __restrict__ conv_bias,
    const float* __restrict__ gates, const float* __restrict__ r_bias, const float* __restrict__ i_bias,
    const float* __restrict__ lam, float c_decay, int C, int bw, int K, float* __restrict__ S_state,
    float* __restrict__ conv_state, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
    T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ float step_s[];  // u [bw] | z [2 bw] | partial sums [teams][2 bw]
  float* u_s = step_s;
  float* z_s = step_s + bw;
  float* part_s = step_s + 3 * bw;
  const int block = blockIdx.x, seq = blockIdx.y;
  const int t = cu_seqlens[seq];
  if (cu_seqlens[seq + 1] <= t) return;
  const size_t slot = (size_t)state_slots[seq];
  const int c0 = block * bw;
  for (int o = threadIdx.x; o < bw; o += blockDim.x) {
    const int c = c0 + o;
    float* state = conv_state + slot * (K - 1) * C + c;  // [K - 1][C], oldest first
    const float x = to_f32(proj[(size_t)t * stride + x_col + c]) + (x_bias ? x_bias[c] : 0.f);
    float acc = conv_bias ? conv_bias[c] : 0.f;
    acc = fmaf(taps[(size_t)c * K + K - 1], x, acc);
    // The same order of additions as the kernel that walks a portion: the current token first, then back.
    for (int j = 1; j < K; ++j) acc = fmaf(taps[(size_t)c * K + (K - 1 - j)], state[(size_t)(K - 1 - j) * C], acc);
    for (int i = 0; i + 1 < K - 1; ++i) state[(size_t)i * C] = state[(size_t)(i + 1) * C];
    if (K > 1) state[(size_t)(K - 2) * C] = x;
    u_s[o] = acc;
  }
  __syncthreads();
  // The maps' products: `teams` threads an output, each over a run of the inputs; the runs' sums are
  // added in their order (the block's size fixes the runs, so a step's arithmetic never depends on
  // which requests it holds).
  const float* g = gates + (size_t)block * bw * 2 * bw;
  const int outputs = 2 * bw;
  const int teams = (int)blockDim.x / outputs > 0 ? (int)blockDim.x / outputs : 1;
  const int per = (bw + teams - 1) / teams;
  for (int item = threadIdx.x; item < teams * outputs; item += blockDim.x) {
    const int team = item / outputs, o = item % outputs;
    const int i0 = team * per, i1 = min(bw, i0 + per);
    float acc = 0.f;
#pragma unroll 8
    for (int i = i0; i < i1; ++i) acc = fmaf(g[(size_t)i * outputs + o], u_s[i], acc);
    part_s[team * outputs + o] = acc;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < outputs; o += blockDim.x) {
    float acc = 0.f;
    for (int team = 0; team < teams; ++team) acc += part_s[team * outputs + o];
    z_s[o] = acc;
  }
  __syncthreads();
  for (int o = threadIdx.x; o < bw; o += blockDim.x) {
    const int c = c0 + o;
    const float r = 1.f / (1.f + expf(-(z_s[o] + r_bias[c])));
    const float i = 1.f / (1.f + expf(-(z_s[bw + o] + i_bias[c])));
    const float l = lam[c];
    const float softplus = fmaxf(l, 0.f) + log1pf(expf(-fabsf(l)));
    const float log_a = -c_decay * r * softplus;
    const float S = fmaf(expf(log_a), S_state[slot * C + c], sqrtf(-expm1f(2.f * log_a)) * i * u_s[o]);
    S_state[slot * C + c] = S;
    const float y = gelu_tanh_f(to_f32(proj[(size_t)t * stride + y_col + c]) + (y_bias ? y_bias[c] : 0.f));
    out[(size_t)t * C + c] = from_f32<T>(S * y);
  }
}

}  // namespace

extern "C" int omnia_rglru_max_taps(void) { return RGLRU_MAX_TAPS; }

// u float32 [tokens, C] = the convolution of this step's inputs (projected columns from x_col plus
// x_bias) continued from conv_state float32 [slots, K - 1, C].
extern "C" int omnia_rglru_conv(const void* proj, int stride, int x_col, const float* x_bias, const float* taps,
                                const float* conv_bias, int C, int K, const float* conv_state, const int* cu_seqlens,
                                const int* state_slots, int num_seqs, float* u, int tokens, int dtype,
                                cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (K < 1 || K > RGLRU_MAX_TAPS || C < 1 || num_seqs < 1) return (int)cudaErrorInvalidValue;
  const int threads = C >= 256 ? 256 : 64;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(rglru_conv_kernel<T>, dim3(tokens, (C + threads - 1) / threads), dim3(threads), 0,
                                          stream, (const T*)proj, stride, x_col, x_bias, taps, conv_bias, C, K, conv_state,
                                          cu_seqlens, state_slots, num_seqs, u)));
  return OMNIA_LAUNCH_RESULT();
}

extern "C" int omnia_rglru_gates(const float* u, const float* z, const float* r_bias, const float* i_bias, const float* lam,
                                 float c_decay, const void* proj, int stride, int y_col, const float* y_bias, int C, int bw,
                                 int tokens, float* a_out, float* b_out, float* y_out, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (bw < 1 || C % bw) return (int)cudaErrorInvalidValue;
  const int threads = C >= 256 ? 256 : 64;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(rglru_gates_kernel<T>, dim3(tokens, (C + threads - 1) / threads), dim3(threads), 0,
                                          stream, u, z, r_bias, i_bias, lam, c_decay, (const T*)proj, stride, y_col, y_bias,
                                          C, bw, tokens, a_out, b_out, y_out)));
  return OMNIA_LAUNCH_RESULT();
}

// out [tokens, C] = S_t y_t in the element type; S_state float32 [slots, C] and conv_state are moved on.
// warps: segments a request's tokens are cut into (1 .. RGLRU_SCAN_WARPS).
extern "C" int omnia_rglru_scan(const float* a, const float* b, const float* y, int C, int K, float* S_state,
                                float* conv_state, const void* proj, int stride, int x_col, const float* x_bias,
                                const int* cu_seqlens, const int* state_slots, int num_seqs, int warps, void* out, int dtype,
                                cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (warps < 1 || warps > RGLRU_SCAN_WARPS || K < 1 || K > RGLRU_MAX_TAPS) return (int)cudaErrorInvalidValue;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(rglru_scan_kernel<T>, dim3((C + 31) / 32, num_seqs), dim3(32 * warps), 0, stream, a,
                                          b, y, C, K, S_state, conv_state, (const T*)proj, stride, x_col, x_bias, cu_seqlens,
                                          state_slots, (T*)out)));
  return OMNIA_LAUNCH_RESULT();
}

// A step of single tokens (cu_seqlens[i + 1] - cu_seqlens[i] is 1, or 0 for a request that sits out):
// everything in one kernel. gates float32 [blocks, bw, 2 bw].
extern "C" int omnia_rglru_step(const void* proj, int stride, int x_col, int y_col, const float* x_bias, const float* y_bias,
                                const float* taps, const float* conv_bias, const float* gates, const float* r_bias,
                                const float* i_bias, const float* lam, float c_decay, int C, int bw, int K, float* S_state,
                                float* conv_state, const int* cu_seqlens, const int* state_slots, int num_seqs, void* out,
                                int dtype, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (bw < 1 || C % bw || K < 1 || K > RGLRU_MAX_TAPS || 5 * bw * sizeof(float) > 40 * 1024) return (int)cudaErrorInvalidValue;
  // Up to eight threads an output of the maps (the products are latency, not arithmetic), 1024 at most.
  int threads = (2 * bw + 31) / 32 * 32;
  if (threads < 1024) threads = threads * 8 <= 1024 ? threads * 8 : 1024 / (2 * bw) > 0 ? 1024 / (2 * bw) * 2 * bw : 1024;
  threads = (threads + 31) / 32 * 32 > 1024 ? 1024 : (threads + 31) / 32 * 32;
  const int teams = threads / (2 * bw) > 0 ? threads / (2 * bw) : 1;
  const size_t smem = (size_t)(3 * bw + teams * 2 * bw) * sizeof(float);
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(rglru_step_kernel<T>, dim3(C / bw, num_seqs), dim3(threads), smem,
                                          stream, (const T*)proj, stride, x_col, y_col, x_bias, y_bias, taps, conv_bias, gates,
                                          r_bias, i_bias, lam, c_decay, C, bw, K, S_state, conv_state, cu_seqlens,
                                          state_slots, (T*)out)));
  return OMNIA_LAUNCH_RESULT();
}
