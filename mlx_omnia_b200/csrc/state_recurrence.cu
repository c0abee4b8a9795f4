// Linear attention as a recurrence over a request's tokens from a float32 state carried in a slot,
// with a decay that is a constant per head or a factor per token, head and key channel:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T      [DK, dv] per head, float32
//   o_t = S_t^T q_t
//
// Three kernels, each taking every constant as an argument:
//
//   inputs      per token, everything that needs no other token, in float32: q and k with the first
//               `rot` dims of every head turned in half-split pairs (i, i + rot / 2) by the angle
//               position * inv_freq[i], then multiplied by q_scale and k_scale; v copied; with decay
//               logits z (float32), a = sigmoid(z + bias)^(1 / tau) = exp(log_sigmoid(z + bias) / tau).
//               Out: one float32 row a token, [q | k | v | a], every section starting on 16 bytes.
//   recurrence  sequential in a request's tokens, parallel over (request, head, run of value columns):
//               the columns of S are independent. A column is held by P threads, each with DK / P of
//               its rows in registers. The block's last STATE_LOADERS threads are loaders: while the
//               column threads walk one run of STATE_CHUNK tokens, the loaders bring the next run's q, k,
//               (a) and v into the other half of a double buffer by asynchronous 16-byte copies; the rows
//               arrive in the layout the column threads read, so nothing is converted on the way, and the
//               column threads issue nothing but the recurrence. One barrier a run.
//               A token's partial sums stay in registers until the run is done: the chain from token to
//               token is one multiply and one fused multiply-add a row. The arithmetic of a token does
//               not depend on how the tokens were cut into steps.
//   heads_out   per token and head: o divided by its root mean square over the head's dv (eps inside the
//               root), times a weight [dv] that the heads share (or none), times silu or sigmoid of the
//               gate's projected columns; rounded once to the element type.
//
//   step        a step in which every request brings one token (decoding) runs all three in one kernel: a
//               block per (request, head) makes its q, k and decays, moves its whole S on (a thread a
//               value column, or a team of threads with the rows dealt out in turn; a team's partial sums
//               are added in the team's order), norms, gates and stores the head's output.
//
// Compiled per key width: -DSTATE_DK=<DK>.
#include "common.cuh"

#ifndef STATE_DK
#define STATE_DK 64
#endif
#define STATE_CHUNK 16     // tokens staged in shared memory at a time
#define STATE_THREADS 448  // column threads of a block at most (with the loaders 512: 128 registers a thread)
#define STATE_LOADERS 64   // threads of a block that stage the next tokens while the others walk these

namespace {

__device__ __forceinline__ int pad4(int n) { return (n + 3) & ~3; }

template <typename T>
__global__ void state_inputs_kernel(const T* __restrict__ proj, int stride, int q_col, int k_col, int v_col, int H, int dv,
                                    const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                                    float q_scale, float k_scale, const float* __restrict__ z, int z_stride,
                                    const float* __restrict__ z_bias, float inv_tau, float* __restrict__ rows,
                                    int row_floats) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DK = STATE_DK;
  __shared__ float cos_s[DK / 2 + 1], sin_s[DK / 2 + 1];
  const size_t t = blockIdx.x;
  const int half = inv_freq != nullptr ? rot / 2 : 0;
  {
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &sin_s[i], &cos_s[i]);
  }
  __syncthreads();
  const T* row = proj + t * stride;
  float* out = rows + t * row_floats;
  const int qk = H * DK, k_at = pad4(qk), v_at = 2 * pad4(qk), a_at = v_at + pad4(H * dv);
  for (int c = threadIdx.x; c < qk; c += blockDim.x) {
    const int i = c % DK;
    float q = to_f32(row[q_col + c]), k = to_f32(row[k_col + c]);
    if (i < 2 * half) {
      const bool low = i < half;
      const int f = low ? i : i - half, other = low ? c + half : c - half;
      const float qo = to_f32(row[q_col + other]), ko = to_f32(row[k_col + other]);
      // (u, v) -> (u cos - v sin, v cos + u sin), u the lower dim of the pair
      q = low ? q * cos_s[f] - qo * sin_s[f] : q * cos_s[f] + qo * sin_s[f];
      k = low ? k * cos_s[f] - ko * sin_s[f] : k * cos_s[f] + ko * sin_s[f];
    }
    out[c] = q * q_scale;
    out[k_at + c] = k * k_scale;
    if (z != nullptr) {
      const float x = z[t * z_stride + c] + (z_bias ? z_bias[c] : 0.f);
      const float log_sigmoid = fminf(x, 0.f) - log1pf(expf(-fabsf(x)));
      out[a_at + c] = expf(log_sigmoid * inv_tau);
    }
  }
  for (int c = threadIdx.x; c < H * dv; c += blockDim.x) out[v_at + c] = to_f32(row[v_col + c]);
}

// CHANNEL: a decay per token and key channel (section a of the rows); else the head's constant.
template <int P, bool CHANNEL>
__global__ void __launch_bounds__(STATE_THREADS + STATE_LOADERS) state_recurrence_kernel(
    const float* __restrict__ rows, int row_floats, int H, int dv, int cols, int parts, int column_threads,
    const float* __restrict__ decay,
    float* __restrict__ S_state, const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots,
    float* __restrict__ o_raw) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DK = STATE_DK;
  constexpr int R = (DK + P - 1) / P;
  // A thread's rows sit in a segment of their own, padded so that the P segments fall on different
  // banks: by four floats when the rows come in fours (segments then start on 16 bytes), else by one.
  constexpr bool FOURS = R % 4 == 0 && DK % 4 == 0;
  constexpr int SEG = FOURS ? R + 4 : R + 1;
  constexpr int VROW = P * SEG;
  constexpr int TC = STATE_CHUNK;
  constexpr int VECS = CHANNEL ? 3 : 2;  // q, k and, per channel, a
  constexpr bool EXACT = P * R == DK;
  extern __shared__ __align__(16) float shared[];
  const int vcols = pad4(cols);
  const int half = TC * (VECS * VROW + vcols);  // floats of one buffer: q | k | (a) [TC][VROW], v [TC][vcols]
  const int head = blockIdx.x / parts, part = blockIdx.x % parts, seq = blockIdx.y;
  const int col0 = part * cols;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  if (end <= begin) return;
  const bool loader = (int)threadIdx.x >= column_threads;
  const int loaders = (int)blockDim.x - column_threads, lt = (int)threadIdx.x - column_threads;
  const int j = threadIdx.x / P, p = threadIdx.x % P;
  const bool live = !loader && j < cols && col0 + j < dv;
  const float lambda = CHANNEL ? 1.f : decay[head];
  const int qk = H * DK, k_at = pad4(qk), v_at = 2 * pad4(qk), a_at = v_at + pad4(H * dv);
  // Whole 16-byte pieces from starts on 16 bytes: the asynchronous way.
  const bool wide = FOURS && cols % 4 == 0 && dv % 4 == 0 && row_floats % 4 == 0;
  constexpr int PIECES = DK / 4 > 0 ? DK / 4 : 1;
  const int per_token = VECS * PIECES + cols / 4;

  auto section = [&](int which) { return which == 0 ? 0 : which == 1 ? k_at : a_at; };
  auto fetch = [&](int t0, int n, float* buf) {
    if (wide) {
      // Item = token * per_token + piece; token and piece are kept up step by step (no division by a
      // number that only the launch knows inside the loop).
      int tok = lt / per_token, piece = lt % per_token;
      for (int item = lt; item < n * per_token; item += loaders) {
        const float* row = rows + (size_t)(t0 + tok) * row_floats;
        const float* src;
        float* dst;
        bool past = false;
        if (piece < VECS * PIECES) {
          const int which = piece / PIECES, i0 = (piece % PIECES) * 4;
          src = row + section(which) + head * DK + i0;
          dst = buf + (which * TC + tok) * VROW + (i0 / R) * SEG + i0 % R;
        } else {
          const int c = (piece - VECS * PIECES) * 4;
          src = row + v_at + head * dv + col0 + c;
          dst = buf + VECS * TC * VROW + tok * vcols + c;
          past = col0 + c >= dv;  // past the head's last column (its last run of columns is a short one)
        }
        if (past) *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        else
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
                       : "memory");
        piece += loaders;
        while (piece >= per_token) piece -= per_token, ++tok;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    } else {
      for (int idx = lt; idx < n * DK; idx += loaders) {
        const int tok = idx / DK, i = idx % DK;
        const float* row = rows + (size_t)(t0 + tok) * row_floats + head * DK + i;
        const int at = tok * VROW + (i / R) * SEG + i % R;
        buf[at] = row[0];
        buf[TC * VROW + at] = row[k_at];
        if (CHANNEL) buf[2 * TC * VROW + at] = row[a_at];
      }
      for (int idx = lt; idx < n * cols; idx += loaders) {
        const int tok = idx / cols, c = idx % cols;
        buf[VECS * TC * VROW + tok * vcols + c] =
            col0 + c < dv ? rows[(size_t)(t0 + tok) * row_floats + v_at + head * dv + col0 + c] : 0.f;
      }
    }
  };

  float S[R];
  float* mine = S_state + (((size_t)state_slots[seq] * H + head) * DK) * dv + col0 + j;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p * R + i;
    S[i] = (live && r < DK) ? mine[(size_t)r * dv] : 0.f;
  }

  const int runs = (end - begin + TC - 1) / TC;
  if (loader) fetch(begin, min(TC, end - begin), shared);
  for (int c = 0; c < runs; ++c) {
    const int t0 = begin + c * TC;
    const int n = min(TC, end - t0);
    if (loader && wide) asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // this run has arrived; the other half has been read
    if (loader) {
      if (c + 1 < runs) fetch(t0 + TC, min(TC, end - t0 - TC), shared + ((c + 1) & 1) * half);
      continue;
    }
    const float* qs = shared + (c & 1) * half;
    const float* ks = qs + TC * VROW;
    const float* as = ks + TC * VROW;
    const float* vs = qs + VECS * TC * VROW;
    float sums[TC];
#pragma unroll
    for (int tok = 0; tok < TC; ++tok) {
      sums[tok] = 0.f;
      if (tok < n) {
        const float* kt = ks + tok * VROW + p * SEG;
        const float* qt = qs + tok * VROW + p * SEG;
        const float* at = as + tok * VROW + p * SEG;
        const float v = live ? vs[tok * vcols + j] : 0.f;
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (FOURS) {
#pragma unroll
          for (int i = 0; i < R; i += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(kt + i), q4 = *reinterpret_cast<const float4*>(qt + i);
            float4 a4 = make_float4(lambda, lambda, lambda, lambda);
            if constexpr (CHANNEL) a4 = *reinterpret_cast<const float4*>(at + i);
            const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w}, aa[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (EXACT || p * R + i + e < DK) {
                S[i + e] = fmaf(kk[e], v, aa[e] * S[i + e]);
                o[e] = fmaf(S[i + e], qq[e], o[e]);
              }
          }
        } else {
#pragma unroll
          for (int i = 0; i < R; ++i)
            if (EXACT || p * R + i < DK) {
              const float a = CHANNEL ? at[i] : lambda;
              S[i] = fmaf(kt[i], v, a * S[i]);
              o[i & 3] = fmaf(S[i], qt[i], o[i & 3]);
            }
        }
        sums[tok] = (o[0] + o[1]) + (o[2] + o[3]);
      }
    }
#pragma unroll
    for (int tok = 0; tok < TC; ++tok)
      if (tok < n) {
        float o = sums[tok];
#pragma unroll
        for (int w = 1; w < P; w <<= 1) o += __shfl_xor_sync(0xffffffffu, o, w);
        if (live && p == 0) o_raw[(size_t)(t0 + tok) * H * dv + head * dv + col0 + j] = o;
      }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p * R + i;
    if (live && r < DK) mine[(size_t)r * dv] = S[i];
  }
}

// A warp per (token, head).
template <typename T>
__global__ void state_heads_out_kernel(const float* __restrict__ o_raw, const T* __restrict__ gate_rows, int gate_stride,
                                       const float* __restrict__ norm_w, float eps, int H, int dv, int tokens, int silu_gate,
                                       T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (size_t)tokens * H) return;
  const size_t t = item / H;
  const int head = (int)(item % H);
  const float* o = o_raw + t * H * dv + head * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += o[c] * o[c];
  const float r = 1.f / sqrtf(warp_sum(ss) / (float)dv + eps);
  for (int c = lane; c < dv; c += 32) {
    const float g = to_f32(gate_rows[t * gate_stride + head * dv + c]);
    const float s = 1.f / (1.f + expf(-g));
    out[t * H * dv + head * dv + c] = from_f32<T>(o[c] * r * (norm_w ? norm_w[c] : 1.f) * (silu_gate ? g * s : s));
  }
}

// grid (heads, requests), STATE_STEP_THREADS threads. Shared: q | k | a [DK] each, partial sums
// [teams][dv], and the block sum's scratch.
#define STATE_STEP_THREADS 1024
template <typename T>
__global__ void __launch_bounds__(STATE_STEP_THREADS) state_step_kernel(
    const T* __restrict__ proj, int stride, int q_col, int k_col, int v_col, int gate_col, int H, int dv,
    const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions, float q_scale, float k_scale,
    const float* __restrict__ z, int z_stride, const float* __restrict__ z_bias, float inv_tau,
    const float* __restrict__ decay, float* __restrict__ S_state, const int* __restrict__ cu_seqlens,
    const int* __restrict__ state_slots, const float* __restrict__ norm_w, float eps, int silu_gate, T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DK = STATE_DK;
  extern __shared__ float step_s[];
  __shared__ float red[33];
  float* q_s = step_s;
  float* k_s = q_s + DK;
  float* a_s = k_s + DK;
  float* part_s = a_s + DK;  // [teams][dv]
  const int head = blockIdx.x, seq = blockIdx.y;
  const size_t t = cu_seqlens[seq];
  if (cu_seqlens[seq + 1] <= (int)t) return;
  const T* row = proj + t * stride;
  const int half = inv_freq != nullptr ? rot / 2 : 0;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < DK; i += blockDim.x) {
    const int c = head * DK + i;
    float q = to_f32(row[q_col + c]), k = to_f32(row[k_col + c]);
    if (i < 2 * half) {
      const bool low = i < half;
      const int f = low ? i : i - half, other = low ? c + half : c - half;
      float sn, cs;
      sincosf(pos * inv_freq[f], &sn, &cs);
      const float qo = to_f32(row[q_col + other]), ko = to_f32(row[k_col + other]);
      q = low ? q * cs - qo * sn : q * cs + qo * sn;
      k = low ? k * cs - ko * sn : k * cs + ko * sn;
    }
    q_s[i] = q * q_scale;
    k_s[i] = k * k_scale;
    if (z != nullptr) {
      const float x = z[t * z_stride + c] + (z_bias ? z_bias[c] : 0.f);
      a_s[i] = expf((fminf(x, 0.f) - log1pf(expf(-fabsf(x)))) * inv_tau);
    } else {
      a_s[i] = decay[head];
    }
  }
  __syncthreads();
  // Thread = (team member, column): member m of `teams` takes rows m, m + teams, ... of its column.
  const int teams = max(1, (int)blockDim.x / dv);
  float* S = S_state + ((size_t)state_slots[seq] * H + head) * DK * dv;
  for (int item = threadIdx.x; item < teams * dv; item += blockDim.x) {
    const int m = item / dv, j = item % dv;
    const float v = to_f32(row[v_col + head * dv + j]);
    float o = 0.f;
#pragma unroll 8
    for (int r = m; r < DK; r += teams) {
      const float s = fmaf(k_s[r], v, a_s[r] * S[(size_t)r * dv + j]);
      S[(size_t)r * dv + j] = s;
      o = fmaf(s, q_s[r], o);
    }
    part_s[m * dv + j] = o;
  }
  __syncthreads();
  float ss = 0.f;
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    float o = 0.f;
    for (int m = 0; m < teams; ++m) o += part_s[m * dv + j];
    part_s[j] = o;  // row 0 of the partial sums becomes the head's output (only this thread reads column j)
    ss += o * o;
  }
  const float r = 1.f / sqrtf(block_sum(ss, red) / (float)dv + eps);
  for (int j = threadIdx.x; j < dv; j += blockDim.x) {
    const float g = to_f32(row[gate_col + head * dv + j]);
    const float sg = 1.f / (1.f + expf(-g));
    out[t * H * dv + head * dv + j] = from_f32<T>(part_s[j] * r * (norm_w ? norm_w[j] : 1.f) * (silu_gate ? g * sg : sg));
  }
}

}  // namespace

extern "C" int omnia_state_dk(void) { return STATE_DK; }

// Floats of a prepared row: [q | k | v | a], sections padded to four floats.
extern "C" int omnia_state_row_floats(int H, int dv, int channel) {
  const int qk = (H * STATE_DK + 3) & ~3, v = (H * dv + 3) & ~3;
  return 2 * qk + v + (channel ? qk : 0);
}

// proj: projected rows [tokens, stride] with q at q_col, k at k_col (H * DK each), v at v_col (H * dv).
// inv_freq: float32 [rot / 2] or null; z: decay logits, float32 [tokens, z_stride] (H * DK used) or null, with
// z_bias float32 [H * DK] or null and inv_tau = 1 / tau. rows: float32 [tokens, row_floats].
extern "C" int omnia_state_inputs(const void* proj, int stride, int q_col, int k_col, int v_col, int H, int dv,
                                  const float* inv_freq, int rot, const int* positions, float q_scale, float k_scale,
                                  const float* z, int z_stride, const float* z_bias, float inv_tau, float* rows,
                                  int tokens, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (H < 1 || dv < 1 || rot < 0 || rot > STATE_DK || rot % 2) return (int)cudaErrorInvalidValue;
  const int row_floats = omnia_state_row_floats(H, dv, z != nullptr);
  const int threads = H * STATE_DK >= 1024 ? 256 : 128;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(state_inputs_kernel<T>, dim3(tokens), dim3(threads), 0, stream, (const T*)proj,
                                          stride, q_col, k_col, v_col, H, dv, inv_freq, rot, positions, q_scale, k_scale,
                                          z, z_stride, z_bias, inv_tau, rows, row_floats)));
  return OMNIA_LAUNCH_RESULT();
}

// The most value columns a block can take: a column needs as many threads as leave each at most 32 rows of S.
extern "C" int omnia_state_max_cols(void) {
  int p = 1;
  while ((STATE_DK + p - 1) / p > 32) p *= 2;
  return STATE_THREADS / p;
}

// rows: the prepared rows; channel != 0: they carry a decay per key channel, else decay float32 [H].
// S_state float32 [slots, H, DK, dv], updated in place; o_raw float32 [tokens, H * dv]. cols: value
// columns a block takes (a head is cut into ceil(dv / cols) runs; at most omnia_state_max_cols());
// column_team: threads a column (1, 2, 4, 8 or 16; 0: chosen here).
extern "C" int omnia_state_recurrence(const float* rows, int H, int dv, int cols, int channel, const float* decay,
                                      float* S_state, const int* cu_seqlens, const int* state_slots, int num_seqs,
                                      float* o_raw, int column_team, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (H < 1 || dv < 1 || cols < 1 || cols > omnia_state_max_cols() || (!channel && decay == nullptr))
    return (int)cudaErrorInvalidValue;
  const int parts = (dv + cols - 1) / cols;
  const int row_floats = omnia_state_row_floats(H, dv, channel);
  const dim3 grid(H * parts, num_seqs);
#define OMNIA_STATE_LAUNCH_AS(P, CHANNEL)                                                                       \
  do {                                                                                                          \
    constexpr int R = (STATE_DK + P - 1) / P;                                                                   \
    constexpr int SEG = (R % 4 == 0 && STATE_DK % 4 == 0) ? R + 4 : R + 1;                                      \
    const size_t smem = sizeof(float) * 2 * STATE_CHUNK * ((size_t)(CHANNEL ? 3 : 2) * P * SEG + ((cols + 3) & ~3)); \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(state_recurrence_kernel<P, CHANNEL>,                           \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return (int)cudaGetLastError();                                                                           \
    const int column_threads = (cols * P + 31) / 32 * 32;                                                       \
    launch_pdl(state_recurrence_kernel<P, CHANNEL>, grid, dim3(column_threads + STATE_LOADERS), smem, stream,    \
               rows, row_floats, H, dv, cols, parts, column_threads, decay, S_state, cu_seqlens, state_slots,   \
               o_raw);                                                                                          \
  } while (0)
#define OMNIA_STATE_LAUNCH(P)                                   \
  do {                                                          \
    if constexpr ((STATE_DK + P - 1) / P <= 32) {               \
      if (channel) OMNIA_STATE_LAUNCH_AS(P, true);              \
      else OMNIA_STATE_LAUNCH_AS(P, false);                     \
    } else {                                                    \
      return (int)cudaErrorInvalidValue;                        \
    }                                                           \
  } while (0)
  // Threads a column (column_team, when the caller names it): as many as give each sixteen rows of S
  // (measured on B200 at key widths of 64 and 128: teams of 4 and 8 walk a prompt a quarter faster
  // than teams of 16; a team's threads read the same q, k and decays as every other column's team, so
  // fewer and longer threads ask shared memory for less), and no more than fit the block.
  if (column_team > 0 && (cols * column_team > STATE_THREADS || column_team > STATE_DK)) return (int)cudaErrorInvalidValue;
  int team = column_team;
  if (team <= 0) {
    team = 1;
    while (team < 16 && STATE_DK / (2 * team) >= 16) team *= 2;
    while ((STATE_DK + team - 1) / team > 32) team *= 2;
    while (team > 1 && cols * team > STATE_THREADS) team /= 2;
  }
  if (team == 16) OMNIA_STATE_LAUNCH(16);
  else if (team == 8) OMNIA_STATE_LAUNCH(8);
  else if (team == 4) OMNIA_STATE_LAUNCH(4);
  else if (team == 2) OMNIA_STATE_LAUNCH(2);
  else if (team == 1 && cols <= STATE_THREADS) OMNIA_STATE_LAUNCH(1);
  else return (int)cudaErrorInvalidValue;
#undef OMNIA_STATE_LAUNCH
#undef OMNIA_STATE_LAUNCH_AS
  return OMNIA_LAUNCH_RESULT();
}

// out [tokens, H * dv] = every head of o_raw divided by its own root mean square (eps inside the root),
// times norm_w [dv] (null: no weight), times silu (silu_gate != 0) or sigmoid of gate_rows[t, :H * dv].
extern "C" int omnia_state_heads_out(const float* o_raw, const void* gate_rows, int gate_stride, const float* norm_w,
                                     float eps, int H, int dv, int tokens, int silu_gate, void* out, int dtype,
                                     cudaStream_t stream) {
  if (tokens == 0) return 0;
  const long long items = (long long)tokens * H;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(state_heads_out_kernel<T>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream,
                                          o_raw, (const T*)gate_rows, gate_stride, norm_w, eps, H, dv, tokens, silu_gate,
                                          (T*)out)));
  return OMNIA_LAUNCH_RESULT();
}

// A step of single tokens (cu_seqlens[i + 1] - cu_seqlens[i] is 1, or 0 for a request that sits out):
// the input step, the recurrence and the heads' norm and gate in one kernel. z float32 or null (then decay).
extern "C" int omnia_state_step(const void* proj, int stride, int q_col, int k_col, int v_col, int gate_col, int H, int dv,
                                const float* inv_freq, int rot, const int* positions, float q_scale, float k_scale,
                                const float* z, int z_stride, const float* z_bias, float inv_tau, const float* decay,
                                float* S_state, const int* cu_seqlens, const int* state_slots, int num_seqs,
                                const float* norm_w, float eps, int silu_gate, void* out, int dtype, cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (H < 1 || dv < 1 || rot < 0 || rot > STATE_DK || rot % 2 || (z == nullptr && decay == nullptr))
    return (int)cudaErrorInvalidValue;
  const int teams = STATE_STEP_THREADS / dv > 0 ? STATE_STEP_THREADS / dv : 1;
  const size_t smem = sizeof(float) * (3 * STATE_DK + (size_t)teams * dv);
  if (smem > 40 * 1024) return (int)cudaErrorInvalidValue;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(state_step_kernel<T>, dim3(H, num_seqs), dim3(STATE_STEP_THREADS), smem, stream,
                                          (const T*)proj, stride, q_col, k_col, v_col, gate_col, H, dv, inv_freq, rot, positions,
                                          q_scale, k_scale, z, z_stride, z_bias, inv_tau, decay, S_state, cu_seqlens,
                                          state_slots, norm_w, eps, silu_gate, (T*)out)));
  return OMNIA_LAUNCH_RESULT();
}
