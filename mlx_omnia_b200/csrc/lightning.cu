// Linear attention with one constant decay per head ("lightning attention"), as a recurrence over a
// request's tokens from a state that is carried in a slot:
//
//   q_t = silu(projected q), k_t = silu(projected k)   [heads, DK]
//   v_t = silu(projected v)                            [heads, dv]
//   S_t = decay_h * S_(t-1) + k_t v_t^T                [DK, dv] per head, float32
//   o_t = S_t^T q_t                                    (no other scale)
//
// followed by one RMS norm over a token's heads side by side with a weight of that size, and a
// sigmoid gate:  out = o / sqrt(mean(o^2) + eps) * w * sigmoid(gate).
//
// The recurrence kernel is sequential in a request's tokens and parallel over (request, head, run
// of value columns): the columns of S are independent. A column is held by P threads (up to 16), each with
// DK / P of its rows in registers. The block's other warps are loaders: while the column threads walk
// one run of LIGHTNING_CHUNK tokens out of shared memory, the loaders fetch the next run's projected
// rows (16 bytes at a time where a head's rows start on 16 bytes and the key width allows), apply the
// activations in float32, round them to the element type, as a product with the activation in its
// epilogue would store them, and leave them in the other half of a double buffer; the two sides meet at
// one barrier a run. A head's q and k are staged once per run of columns, so a block with few columns
// spends most of its instructions there: what the loaders do per element decides the kernel's pace. A token's partial sums stay in registers until its run is done,
// so the shuffles that add them up are off the chain from token to token, which is one fused
// multiply-add a row. The state, the decay and every sum stay float32. It serves decode steps (one
// token a request) and prompts' portions of any length alike; the order of a column's additions does
// not depend on how a prompt was cut.
//
// Compiled per key width: -DLIGHTNING_DK=<DK>.
#include "common.cuh"

#ifndef LIGHTNING_DK
#define LIGHTNING_DK 64
#endif
#define LIGHTNING_CHUNK 16     // tokens staged in shared memory at a time
#define LIGHTNING_LOADERS 128  // threads of a block that stage the next tokens while the others walk these
#define LIGHTNING_THREADS 512  // of a block at most: 128 registers a thread for the state's rows

namespace {

// SiLU in float32. The 16-bit types take the fast exponential and division that the products' fused
// epilogues take (the result is rounded to 8 bits of mantissa next), float32 the exact ones.
template <typename T>
__device__ __forceinline__ float silu_as(float x) {
  if constexpr (sizeof(T) == 2) return __fdividef(x, 1.f + __expf(-x));
  else return x / (1.f + expf(-x));
}

template <typename T, int P>
__global__ void __launch_bounds__(LIGHTNING_THREADS) lightning_recurrence_kernel(
    const T* __restrict__ proj, int stride, int q_col, int k_col, int v_col, int H, int dv, int cols, int parts,
    int column_threads, const float* __restrict__ decay, float* __restrict__ S_state,
    const int* __restrict__ cu_seqlens, const int* __restrict__ state_slots, float* __restrict__ o_raw) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int DK = LIGHTNING_DK;
  constexpr int R = (DK + P - 1) / P;
  // A thread's rows sit in a segment of their own, padded so that the P segments fall on different
  // banks: by four floats when the rows come in fours (segments then start on 16 bytes and are read
  // and written four floats at a time), else by one.
  constexpr bool FOURS = R % 4 == 0;
  constexpr int SEG = FOURS ? R + 4 : R + 1;
  constexpr int VROW = P * SEG;  // floats of one token's vector of DK
  constexpr int TC = LIGHTNING_CHUNK;
  constexpr int VEC = 16 / (int)sizeof(T);  // elements in 16 bytes of a projected row
  constexpr bool EXACT = P * R == DK;       // every thread's R rows are rows of S: nothing to guard
  extern __shared__ __align__(16) float shared[];
  const int half = 2 * TC * VROW + TC * cols;  // floats of one buffer: q [TC][VROW] | k [TC][VROW] | v [TC][cols]
  const int head = blockIdx.x / parts, part = blockIdx.x % parts, seq = blockIdx.y;
  const int col0 = part * cols;
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  if (end <= begin) return;
  const bool loader = (int)threadIdx.x >= column_threads;
  const int loaders = (int)blockDim.x - column_threads, lt = (int)threadIdx.x - column_threads;
  const int j = threadIdx.x / P, p = threadIdx.x % P;
  const bool live = !loader && j < cols && col0 + j < dv;
  const float lambda = decay[head];
  // Whether this block's q, k and v can be fetched 16 bytes at a time: whole pieces, every row's start on 16 bytes.
  const bool wide = FOURS && DK % VEC == 0 && cols % VEC == 0 && (stride * sizeof(T)) % 16 == 0 &&
                    (reinterpret_cast<uintptr_t>(proj + q_col + head * DK) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(proj + k_col + head * DK) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(proj + v_col + head * dv + col0) & 15) == 0;
  constexpr int PIECES = DK / VEC > 0 ? DK / VEC : 1;  // 16-byte pieces of a head's q (and k) row
  const int v_pieces = cols / VEC, per_token = 2 * PIECES + v_pieces;
  uint4* raw = reinterpret_cast<uint4*>(shared + 2 * half);  // [TC * per_token] pieces as they come from memory

  // The wide way has two steps a run. `fetch` starts the copies of tokens [t0, t0 + n) into `raw`
  // (asynchronous copies: the thread goes on at once); `cook` waits for this thread's own copies, applies
  // the activations in float32, rounds to the element type and lays the floats out for the column
  // threads. A thread cooks exactly the pieces it fetched, so the loaders need no barrier of their own,
  // and the copies of one run are in flight while the run before it is walked.
  auto fetch = [&](int t0, int n) {
    for (int item = lt; item < n * per_token; item += loaders) {
      const int tok = item / per_token, r = item % per_token;
      const T* row = proj + (size_t)(t0 + tok) * stride;
      const T* src = r < PIECES       ? row + q_col + head * DK + r * VEC
                     : r < 2 * PIECES ? row + k_col + head * DK + (r - PIECES) * VEC
                                      : row + v_col + head * dv + col0 + (r - 2 * PIECES) * VEC;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(raw + item)), "l"(src)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto cook = [&](int n, float* buf) {
    float* qs = buf;
    float* ks = buf + TC * VROW;
    float* vs = ks + TC * VROW;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    for (int item = lt; item < n * per_token; item += loaders) {
      const int tok = item / per_token, r = item % per_token;
      const uint4 piece = raw[item];
      float x[VEC];
      if constexpr (sizeof(T) == 4) {
        x[0] = __uint_as_float(piece.x), x[1] = __uint_as_float(piece.y), x[2] = __uint_as_float(piece.z),
        x[3] = __uint_as_float(piece.w);
      } else {
        const T* e = reinterpret_cast<const T*>(&piece);
#pragma unroll
        for (int i = 0; i < VEC; ++i) x[i] = to_f32(e[i]);
      }
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] = to_f32(from_f32<T>(silu_as<T>(x[e])));
      float* dst;
      if (r < 2 * PIECES) {
        const int i0 = (r < PIECES ? r : r - PIECES) * VEC;
        dst = (r < PIECES ? qs : ks) + tok * VROW + (i0 / R) * SEG + i0 % R;  // VEC divides R or R divides VEC's fours
        if constexpr (VEC == 8 && R % 8 != 0) {
          // The second four floats may belong to the next segment.
          const int i1 = i0 + 4;
          *reinterpret_cast<float4*>(dst) = make_float4(x[0], x[1], x[2], x[3]);
          dst = (r < PIECES ? qs : ks) + tok * VROW + (i1 / R) * SEG + i1 % R;
          *reinterpret_cast<float4*>(dst) = make_float4(x[4], x[5], x[6], x[7]);
          continue;
        }
      } else {
        dst = vs + tok * cols + (r - 2 * PIECES) * VEC;
      }
#pragma unroll
      for (int e = 0; e < VEC; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(x[e], x[e + 1], x[e + 2], x[e + 3]);
    }
  };

  // The plain way: tokens [t0, t0 + n) into buffer `buf`, element by element.
  auto stage = [&](int t0, int n, float* buf) {
    float* qs = buf;
    float* ks = buf + TC * VROW;
    float* vs = ks + TC * VROW;
#pragma unroll 4
    for (int idx = lt; idx < n * DK; idx += loaders) {
      const int tok = idx / DK, i = idx % DK;
      const T* src = proj + (size_t)(t0 + tok) * stride + head * DK + i;
      const float q = to_f32(src[q_col]), k = to_f32(src[k_col]);
      const int at = tok * VROW + (i / R) * SEG + i % R;
      qs[at] = to_f32(from_f32<T>(silu_as<T>(q)));
      ks[at] = to_f32(from_f32<T>(silu_as<T>(k)));
    }
#pragma unroll 4
    for (int idx = lt; idx < n * cols; idx += loaders) {
      const int tok = idx / cols, c = idx % cols;
      vs[idx] = col0 + c < dv
                    ? to_f32(from_f32<T>(silu_as<T>(to_f32(proj[(size_t)(t0 + tok) * stride + v_col + head * dv + col0 + c]))))
                    : 0.f;
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
  if (loader) {
    if (wide) {
      fetch(begin, min(TC, end - begin));
      cook(min(TC, end - begin), shared);
      if (runs > 1) fetch(begin + TC, min(TC, end - begin - TC));
    } else {
      stage(begin, min(TC, end - begin), shared);
    }
  }
  __syncthreads();
  for (int c = 0; c < runs; ++c) {
    const int t0 = begin + c * TC;
    const int n = min(TC, end - t0);
    if (loader) {
      if (c + 1 < runs) {
        if (wide) {
          cook(min(TC, end - t0 - TC), shared + ((c + 1) & 1) * half);
          if (c + 2 < runs) fetch(t0 + 2 * TC, min(TC, end - t0 - 2 * TC));
        } else {
          stage(t0 + TC, min(TC, end - t0 - TC), shared + ((c + 1) & 1) * half);
        }
      }
    } else {
      const float* qs = shared + (c & 1) * half;
      const float* ks = qs + TC * VROW;
      const float* vs = ks + TC * VROW;
      float sums[TC];
#pragma unroll
      for (int tok = 0; tok < TC; ++tok) {
        sums[tok] = 0.f;
        if (tok < n) {
          const float* kt = ks + tok * VROW + p * SEG;
          const float* qt = qs + tok * VROW + p * SEG;
          const float v = live ? vs[tok * cols + j] : 0.f;
          // Four partial sums, so that a token's dot product is four short chains instead of one of R.
          float o[4] = {0.f, 0.f, 0.f, 0.f};
          if constexpr (FOURS) {
#pragma unroll
            for (int i = 0; i < R; i += 4) {
              const float4 k4 = *reinterpret_cast<const float4*>(kt + i), q4 = *reinterpret_cast<const float4*>(qt + i);
              const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (EXACT || p * R + i + e < DK) {
                  S[i + e] = fmaf(kk[e], v, lambda * S[i + e]);
                  o[e] = fmaf(S[i + e], qq[e], o[e]);
                }
            }
          } else {
#pragma unroll
            for (int i = 0; i < R; ++i)
              if (EXACT || p * R + i < DK) {
                S[i] = fmaf(kt[i], v, lambda * S[i]);
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
    __syncthreads();  // the next run is staged, this one has been read
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int r = p * R + i;
    if (live && r < DK) mine[(size_t)r * dv] = S[i];
  }
}

// out[t] = o[t] / sqrt(mean(o[t]^2) + eps) * w * sigmoid(gate[t]) over a token's whole row of
// `width` = heads * dv; a block per token.
template <typename T>
__global__ void lightning_out_kernel(const float* __restrict__ o_raw, const T* __restrict__ gate_rows, int gate_stride,
                                     const float* __restrict__ norm_w, float eps, int width, T* __restrict__ out) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float red[33];
  const size_t t = blockIdx.x;
  const float* o = o_raw + t * width;
  float ss = 0.f;
  for (int c = threadIdx.x; c < width; c += blockDim.x) ss += o[c] * o[c];
  const float r = rsqrtf(block_sum(ss, red) / (float)width + eps);
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    const float gate = to_f32(gate_rows[t * gate_stride + c]);
    out[t * width + c] = from_f32<T>(o[c] * r * norm_w[c] / (1.f + expf(-gate)));
  }
}

}  // namespace

extern "C" int omnia_lightning_dk(void) { return LIGHTNING_DK; }

// proj: the projected rows [tokens, stride] with q at q_col, k at k_col (heads * DK each) and v at
// v_col (heads * dv); decay float32 [heads]; S_state float32 [slots, heads, DK, dv], updated in place;
// o_raw float32 [tokens, heads * dv] receives the unnormed outputs. parts: runs of columns a head is
// cut into (dv must divide into them; a run of at most 384 columns, 96 for four threads a column).
extern "C" int omnia_lightning_recurrence(const void* proj, int stride, int q_col, int k_col, int v_col, int H, int dv,
                                          int parts, const float* decay, float* S_state, const int* cu_seqlens,
                                          const int* state_slots, int num_seqs, float* o_raw, int dtype,
                                          cudaStream_t stream) {
  if (num_seqs == 0) return 0;
  if (H < 1 || dv < 1 || parts < 1 || dv % parts != 0) return (int)cudaErrorInvalidValue;
  const int cols = dv / parts;
  const dim3 grid(H * parts, num_seqs);
#define OMNIA_LIGHTNING_LAUNCH(P)                                                                              \
  do {                                                                                                         \
    constexpr int R = (LIGHTNING_DK + P - 1) / P;                                                              \
    const size_t smem = sizeof(float) * 2 * ((size_t)2 * LIGHTNING_CHUNK * P * (R % 4 == 0 ? R + 4 : R + 1) + LIGHTNING_CHUNK * cols) + \
                        (size_t)LIGHTNING_CHUNK * (2 * (LIGHTNING_DK * sizeof(T) / 16 + 1) + cols * sizeof(T) / 16 + 1) * 16; \
    if (smem > 48 * 1024 && cudaFuncSetAttribute(lightning_recurrence_kernel<T, P>,                            \
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
      return (int)cudaGetLastError();                                                                          \
    const int column_threads = (cols * P + 31) / 32 * 32;                                                      \
    launch_pdl(lightning_recurrence_kernel<T, P>, grid, dim3(column_threads + LIGHTNING_LOADERS), smem, stream, \
               (const T*)proj, stride, q_col, k_col, v_col, H, dv, cols, parts, column_threads, decay, S_state, \
               cu_seqlens, state_slots, o_raw);                                                                \
  } while (0)
  // Threads a column: as many as leave each at least four rows of S and fit the block. A column's
  // threads share out its rows, so more of them shorten what a token costs a warp; their partial sums
  // meet in shuffles after a run of tokens, off the chain from token to token.
  constexpr int ROOM = LIGHTNING_THREADS - LIGHTNING_LOADERS;  // threads left for the columns
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (cols * 16 <= ROOM && LIGHTNING_DK >= 64) OMNIA_LIGHTNING_LAUNCH(16);
    else if (cols * 8 <= ROOM && LIGHTNING_DK >= 32) OMNIA_LIGHTNING_LAUNCH(8);
    else if (cols * 4 <= ROOM && LIGHTNING_DK >= 16) OMNIA_LIGHTNING_LAUNCH(4);
    else if (cols * 2 <= ROOM && LIGHTNING_DK >= 8) OMNIA_LIGHTNING_LAUNCH(2);
    else if (cols <= ROOM) OMNIA_LIGHTNING_LAUNCH(1);
    else return (int)cudaErrorInvalidValue;
  });
#undef OMNIA_LIGHTNING_LAUNCH
  return OMNIA_LAUNCH_RESULT();
}

// out [tokens, width] = o_raw normed over the whole row (weight norm_w [width], eps) times
// sigmoid(gate_rows[t, :width]) (rows gate_stride apart).
extern "C" int omnia_lightning_out(const float* o_raw, const void* gate_rows, int gate_stride, const float* norm_w,
                                   float eps, int width, int tokens, void* out, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  const int threads = width >= 1024 ? 256 : 128;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(lightning_out_kernel<T>, dim3(tokens), dim3(threads), 0, stream, o_raw,
                                          (const T*)gate_rows, gate_stride, norm_w, eps, width, (T*)out)));
  return OMNIA_LAUNCH_RESULT();
}
