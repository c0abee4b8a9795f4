// A routed mixture of small gated feed-forward layers ("experts"), as kernels that never ask the
// host which token went where:
//
//   route     per token: router logits in float32, softmax over all router outputs, choice by
//             score + correction, the `top` largest; the weights are the scores themselves. Router
//             outputs at or beyond `experts` name identity experts (they have no tensors).
//   plan      one block: where each expert's rows begin in the sorted order, and the list of row
//             tiles (expert, first row, rows) that the grouped products walk.
//   scatter   per (token, choice): its place among its expert's rows.
//   grouped products over the sorted rows, a tile of rows belonging to one expert:
//             act = silu(h W_gate^T) * (h W_up^T) (the rows of h gathered through the sorted order),
//             then out = act W_down^T.
//   combine   per token: the weighted sum of its choices' rows in a fixed order (identity experts
//             add the token's own input), rounded once.
//
// The products have two forms: float32 arithmetic on the ordinary cores for any element type (the
// 32-bit path), and bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulation).
#include "common.cuh"

#include <limits.h>

namespace {

constexpr int TILE_ROWS = 64;  // rows of a tile of the grouped products

// What an expert does with its gate and up values: silu(gate) * up, or with limit > 0 the clamped
// unit g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(alpha * g) * (u + 1).
__device__ __forceinline__ float gated_unit(float gate, float up, float alpha, float limit) {
  if (limit > 0.f) {
    const float g = fminf(gate, limit), u = fminf(fmaxf(up, -limit), limit);
    return g / (1.f + expf(-alpha * g)) * (u + 1.f);
  }
  return gate / (1.f + expf(-gate)) * up;
}

// ---------------------------------------------------------------------------------
// A block routes TOK consecutive tokens (8 where there are many: every router row is then fetched
// once for eight tokens instead of once a token; 1 in a small step, which wants warps, not reuse).
// The tokens' rows wait in shared memory as float32; a warp owns every eighth router output and takes
// the dot products of CHUNK of them with all TOK rows in one pass over the columns.
// Then warp t finishes token t: softmax over all outputs, choice scores, the `top` largest.
template <typename T, int TOK, int THREADS, int CHUNK>
__global__ void __launch_bounds__(THREADS)
moe_route_kernel(const T* __restrict__ h, const float* __restrict__ router, const float* __restrict__ correction,
                 int tokens, int outputs, int experts, int hidden, int top, int sigmoid_scores,
                 int* __restrict__ choice, float* __restrict__ weight, int* __restrict__ counts) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int WARPS = THREADS / 32;
  static_assert(TOK <= WARPS, "a warp finishes a token");
  extern __shared__ __align__(16) float route_s[];
  const int padded = (outputs + 3) / 4 * 4;
  float* hrow = route_s;                           // [TOK][hidden]
  float* scores = hrow + (size_t)TOK * hidden;     // [TOK][padded] logits, then scores; [TOK][padded] choice scores
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * TOK, live = min(TOK, tokens - t0);
  for (int tok = 0; tok < TOK; ++tok)
    for (int i = threadIdx.x; i < hidden; i += THREADS)
      hrow[(size_t)tok * hidden + i] = tok < live ? to_f32(h[(size_t)(t0 + tok) * hidden + i]) : 0.f;
  __syncthreads();
  // CHUNK router outputs a warp at a time (outputs warp, warp + WARPS, ...): a lane reads a float4 of
  // each token's row once and uses it against all of them, and the CHUNK loads of the router's rows,
  // times the unrolling, are in flight together. (A single token: 32 warps, an output each, eight
  // steps of the columns in flight: the router's rows come from memory, and the block is their latency.)
  const bool wide = (hidden & 3) == 0 && ((uintptr_t)router & 15) == 0;
  for (int e0 = warp; e0 < outputs; e0 += WARPS * CHUNK) {
    float acc[CHUNK][TOK];
#pragma unroll
    for (int c = 0; c < CHUNK; ++c)
#pragma unroll
      for (int tok = 0; tok < TOK; ++tok) acc[c][tok] = 0.f;
    if (wide) {
      const int quads = hidden / 4;
      const float4* w4 = reinterpret_cast<const float4*>(router);
      const float4* h4 = reinterpret_cast<const float4*>(hrow);
#pragma unroll(CHUNK == 1 ? 8 : 2)
      for (int q = lane; q < quads; q += 32) {
        float4 b[CHUNK];
#pragma unroll
        for (int c = 0; c < CHUNK; ++c) {
          const int e = e0 + c * WARPS;
          b[c] = e < outputs ? __ldg(w4 + (size_t)e * quads + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int tok = 0; tok < TOK; ++tok) {
          const float4 a = h4[(size_t)tok * quads + q];
#pragma unroll
          for (int c = 0; c < CHUNK; ++c) acc[c][tok] += a.x * b[c].x + a.y * b[c].y + a.z * b[c].z + a.w * b[c].w;
        }
      }
    } else {
      for (int i = lane; i < hidden; i += 32)
#pragma unroll
        for (int c = 0; c < CHUNK; ++c) {
          const int e = e0 + c * WARPS;
          const float b = e < outputs ? router[(size_t)e * hidden + i] : 0.f;
#pragma unroll
          for (int tok = 0; tok < TOK; ++tok) acc[c][tok] += hrow[(size_t)tok * hidden + i] * b;
        }
    }
#pragma unroll
    for (int c = 0; c < CHUNK; ++c)
#pragma unroll
      for (int tok = 0; tok < TOK; ++tok) {
        const float v = warp_sum(acc[c][tok]);
        const int e = e0 + c * WARPS;
        if (lane == 0 && e < outputs) scores[(size_t)tok * padded + e] = v;
      }
  }
  __syncthreads();
  if (warp >= live) return;
  const int t = t0 + warp;
  float* score = scores + (size_t)warp * padded;
  float* pick = scores + (size_t)(TOK + warp) * padded;
  float top_z = -INFINITY;
  for (int e = lane; e < outputs; e += 32) top_z = fmaxf(top_z, score[e]);
  top_z = warp_max(top_z);
  float sum = 0.f;
  for (int e = lane; e < outputs; e += 32) sum += expf(score[e] - top_z);
  sum = warp_sum(sum);
  for (int e = lane; e < outputs; e += 32) {
    // Every output's score by itself (a sigmoid), or its share among all outputs (a softmax).
    const float s = sigmoid_scores ? 1.f / (1.f + expf(-score[e])) : expf(score[e] - top_z) / sum;
    score[e] = s;
    pick[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    // The largest choice score not taken yet; of equal ones the lowest index. A row of NaNs still
    // gets `top` different experts (the lowest indices).
    float best = -INFINITY;
    int best_e = INT_MAX, spare = INT_MAX;
    for (int e = lane; e < outputs; e += 32) {
      const float v = pick[e];
      if (v == -INFINITY) continue;  // taken
      spare = min(spare, e);
      if (v > best || (v == best && e < best_e)) best = v, best_e = e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      spare = min(spare, __shfl_xor_sync(0xffffffffu, spare, o));
      if (other > best || (other == best && other_e < best_e)) best = other, best_e = other_e;
    }
    if (best_e == INT_MAX) best_e = spare;
    if (lane == 0) {
      choice[(size_t)t * top + k] = best_e;
      weight[(size_t)t * top + k] = score[best_e];
      if (best_e < experts) atomicAdd(counts + best_e, 1);
      pick[best_e] = -INFINITY;
    }
    __syncwarp();
  }
}

// ---------------------------------------------------------------------------------
// offsets [experts + 1]; tiles [max_tiles, 3] = (expert, first row, rows); tile_count [1];
// counts and cursors are left zero for the launches that follow.
// With `choice` given (a small step) the one block goes on to place every (token, choice) itself, which
// saves the launch of the scatter kernel below.
__global__ void moe_plan_kernel(int* __restrict__ counts, int* __restrict__ cursors, int* __restrict__ offsets,
                                int* __restrict__ tiles, int* __restrict__ tile_count, int experts, int max_tiles,
                                int tile_rows, const int* __restrict__ choice, int* __restrict__ place,
                                int* __restrict__ source, int pairs, int top) {
  pdl_wait();
  pdl_launch_dependents();
  extern __shared__ int plan_s[];  // [experts + 1] row offsets, [experts + 1] tile offsets
  int* row0 = plan_s;
  int* tile0 = plan_s + experts + 1;
  if (threadIdx.x == 0) {
    int rows = 0, listed = 0;
    for (int e = 0; e < experts; ++e) {
      row0[e] = rows, tile0[e] = listed;
      rows += counts[e];
      listed += (counts[e] + tile_rows - 1) / tile_rows;
    }
    row0[experts] = rows, tile0[experts] = listed;
    *tile_count = min(listed, max_tiles);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = row0[e];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int rows = row0[e + 1] - row0[e];
    for (int i = 0, at = tile0[e]; i * tile_rows < rows && at < max_tiles; ++i, ++at) {
      tiles[3 * at] = e;
      tiles[3 * at + 1] = row0[e] + i * tile_rows;
      tiles[3 * at + 2] = min(tile_rows, rows - i * tile_rows);
    }
    counts[e] = 0;
    cursors[e] = 0;
  }
  if (choice == nullptr) return;
  __syncthreads();  // the cursors are zero (this block is the only one that touches them)
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = choice[i];
    if (e >= experts) {
      place[i] = -1;
    } else {
      const int row = row0[e] + atomicAdd(cursors + e, 1);
      place[i] = row;
      source[row] = i / top;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursors[e] = 0;
}

// ---------------------------------------------------------------------------------
// place[t * top + k] = the sorted row of the choice (-1: an identity expert); source[row] = t.
__global__ void moe_scatter_kernel(const int* __restrict__ choice, const int* __restrict__ offsets,
                                   int* __restrict__ cursors, int* __restrict__ place, int* __restrict__ source,
                                   int pairs, int top, int experts) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= pairs) return;
  const int e = choice[i];
  if (e >= experts) {
    place[i] = -1;
    return;
  }
  const int row = offsets[e] + atomicAdd(cursors + e, 1);
  place[i] = row;
  source[row] = i / top;
}

// ---------------------------------------------------------------------------------
// Grouped product on the ordinary cores, any element type, float32 arithmetic.
//   a:     [rows, k]; row r of the sorted order reads a[source ? source[r] : r]
//   w:     [experts, n_total, k]; DUAL: n_total = 2 n, gate rows then up rows
//   out:   [sorted rows, n]; DUAL: silu(gate) * up
// grid (max tiles, n / 64): a block owns 64 rows x 64 columns, 256 threads of 4 x 4.
template <typename T, bool DUAL>
__global__ void __launch_bounds__(256)
moe_product_kernel(const T* __restrict__ a, const int* __restrict__ source, const T* __restrict__ w,
                   T* __restrict__ out, const int* __restrict__ tiles, const int* __restrict__ tile_count,
                   int n, int k, float alpha, float limit) {
  pdl_wait();
  pdl_launch_dependents();
  if ((int)blockIdx.x >= *tile_count) return;
  constexpr int BK = 16;
  __shared__ float As[BK][TILE_ROWS + 4], Bs[DUAL ? 2 : 1][BK][64 + 4];
  __shared__ int src_row[TILE_ROWS];
  const int expert = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * 64;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  if (tid < TILE_ROWS) src_row[tid] = tid < rows ? (source ? source[row0 + tid] : row0 + tid) : -1;
  __syncthreads();
  const T* we = w + (size_t)expert * (DUAL ? 2 : 1) * n * k;
  float acc[DUAL ? 2 : 1][4][4];
#pragma unroll
  for (int d = 0; d < (DUAL ? 2 : 1); ++d)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[d][i][j] = 0.f;
  for (int k0 = 0; k0 < k; k0 += BK) {
    for (int i = tid; i < TILE_ROWS * BK; i += 256) {
      const int r = i / BK, c = i % BK;
      const int src = src_row[r];
      As[c][r] = (src >= 0 && k0 + c < k) ? to_f32(a[(size_t)src * k + k0 + c]) : 0.f;
    }
    for (int i = tid; i < 64 * BK; i += 256) {
      const int r = i / BK, c = i % BK;
      const bool live = n0 + r < n && k0 + c < k;
      Bs[0][c][r] = live ? to_f32(we[(size_t)(n0 + r) * k + k0 + c]) : 0.f;
      if (DUAL) Bs[1][c][r] = live ? to_f32(we[(size_t)(n + n0 + r) * k + k0 + c]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float av[4], bv[DUAL ? 2 : 1][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int d = 0; d < (DUAL ? 2 : 1); ++d)
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[d][j] = Bs[d][kk][tx * 4 + j];
#pragma unroll
      for (int d = 0; d < (DUAL ? 2 : 1); ++d)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[d][i][j] += av[i] * bv[d][j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = n0 + tx * 4 + j;
      if (c >= n) continue;
      float v = acc[0][i][j];
      if (DUAL) v = gated_unit(v, acc[1][i][j], alpha, limit);
      out[(size_t)(row0 + r) * n + c] = from_f32<T>(v);
    }
  }
}

// ---------------------------------------------------------------------------------
// The same grouped product in bfloat16 on the tensor cores. A block of four warps owns 64 rows x 64
// columns; a warp 16 rows x 64 columns (x 2 with DUAL). Steps of 32 along k through a cp.async
// double buffer; k % 8 == 0 and operands whose rows start on 16 bytes.
typedef __nv_bfloat16 bf16;

// A 16-byte asynchronous copy to a shared-memory address; not valid: the 16 bytes are zero-filled.
__device__ __forceinline__ void cp_async16_to(uint32_t smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const bf16* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

constexpr int TC_BK = 32, TC_ROW = TC_BK + 8, TC_STAGES = 4;
constexpr size_t tc_smem_bytes(bool dual) {
  return (size_t)TC_STAGES * (TILE_ROWS + (dual ? 2 : 1) * 64) * TC_ROW * sizeof(__nv_bfloat16);
}

template <bool DUAL>
__global__ void __launch_bounds__(128)
moe_product_tc_kernel(const bf16* __restrict__ a, const int* __restrict__ source, const bf16* __restrict__ w,
                      bf16* __restrict__ out, const int* __restrict__ tiles, const int* __restrict__ tile_count,
                      int n, int k, float alpha, float limit) {
  pdl_wait();
  pdl_launch_dependents();
  if ((int)blockIdx.x >= *tile_count) return;
  constexpr int BK = TC_BK, ROW = TC_ROW, PARTS = DUAL ? 2 : 1, STAGES = TC_STAGES;
  extern __shared__ __align__(16) unsigned char tc_smem[];
  typedef bf16 (*ATiles)[TILE_ROWS][ROW];
  typedef bf16 (*BTiles)[PARTS][64][ROW];
  ATiles As = reinterpret_cast<ATiles>(tc_smem);                                                  // [STAGES][64][ROW]
  BTiles Bs = reinterpret_cast<BTiles>(tc_smem + (size_t)STAGES * TILE_ROWS * ROW * sizeof(bf16));  // [STAGES][PARTS][64][ROW]
  __shared__ int src_row[TILE_ROWS];
  const int expert = tiles[3 * blockIdx.x], row0 = tiles[3 * blockIdx.x + 1], rows = tiles[3 * blockIdx.x + 2];
  const int n0 = blockIdx.y * 64;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < TILE_ROWS) src_row[tid] = tid < rows ? (source ? source[row0 + tid] : row0 + tid) : -1;
  __syncthreads();
  const bf16* we = w + (size_t)expert * PARTS * n * k;
  // A stage is 64 rows x 4 chunks of 16 bytes of A and of each part of B: a thread copies two chunks of
  // each (rows tid / 4 and 32 + tid / 4, chunk tid % 4), and where they come from and go to is worked out
  // once: a step of the loop is then a copy, an add and a test a chunk. (With one or two rows a tile the
  // kernel is a stream of weights that the issue of its own instructions bounds: 2.6 TB/s with the
  // addresses recomputed every step.) Rows of A beyond the tile's own are not copied at all: a row of
  // the product depends on its own row of A only, and theirs is never stored.
  constexpr uint32_t A_STAGE = TILE_ROWS * ROW * sizeof(bf16), B_STAGE = PARTS * 64 * ROW * sizeof(bf16);
  const int chunk = (tid & 3) * 8;
  const bf16* a_src[2];
  const bf16* b_src[2][PARTS];
  uint32_t a_dst[2], b_dst[2][PARTS];
  bool a_on[2], b_on[2];
#pragma unroll
  for (int slot = 0; slot < 2; ++slot) {
    const int r = slot * 32 + (tid >> 2);
    const int src = src_row[r];
    a_on[slot] = src >= 0;
    a_src[slot] = a + (size_t)(src >= 0 ? src : 0) * k + chunk;
    a_dst[slot] = (uint32_t)__cvta_generic_to_shared(&As[0][r][chunk]);
    b_on[slot] = n0 + r < n;
#pragma unroll
    for (int part = 0; part < PARTS; ++part) {
      b_src[slot][part] = we + (size_t)(part * n + (b_on[slot] ? n0 + r : 0)) * k + chunk;
      b_dst[slot][part] = (uint32_t)__cvta_generic_to_shared(&Bs[0][part][r][chunk]);
    }
  }
  auto load = [&](int k0, int stage) {
    const bool in_k = k0 + chunk < k;
#pragma unroll
    for (int slot = 0; slot < 2; ++slot) {
      if (a_on[slot]) cp_async16_to(a_dst[slot] + stage * A_STAGE, a_src[slot] + k0, in_k);
#pragma unroll
      for (int part = 0; part < PARTS; ++part)
        cp_async16_to(b_dst[slot][part] + stage * B_STAGE, b_src[slot][part] + k0, b_on[slot] && in_k);
    }
  };
  float acc[PARTS][8][4];
#pragma unroll
  for (int part = 0; part < PARTS; ++part)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[part][j][0] = acc[part][j][1] = acc[part][j][2] = acc[part][j][3] = 0.f;
  const int steps = (k + BK - 1) / BK;
  // A ring of STAGES stages, STAGES - 1 of them on their way at any time: a block with one or two rows
  // (a decode step) is a stream of weights, and what bounds it is how much of the stream is in flight.
#pragma unroll
  for (int s0 = 0; s0 < STAGES - 1; ++s0) {
    if (s0 < steps) load(s0 * BK, s0);
    cp_async_commit();
  }
  const int mat = lane >> 3;
  const bool busy = warp * 16 < rows;  // a warp none of whose 16 rows is the tile's own only helps to load
  for (int step = 0; step < steps; ++step) {
    cp_async_wait<STAGES - 2>();
    __syncthreads();  // stage `step` has landed, and everyone is done with the stage that is filled next
    if (step + STAGES - 1 < steps) load((step + STAGES - 1) * BK, (step + STAGES - 1) % STAGES);
    cp_async_commit();
    const int stage = step % STAGES;
    if (!busy) continue;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      unsigned af[4];
      ldmatrix_x4(af[0], af[1], af[2], af[3], &As[stage][warp * 16 + (mat & 1) * 8 + (lane & 7)][ks * 16 + (mat >> 1) * 8]);
#pragma unroll
      for (int part = 0; part < PARTS; ++part)
#pragma unroll
        for (int j2 = 0; j2 < 4; ++j2) {
          unsigned b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, &Bs[stage][part][j2 * 16 + (mat >> 1) * 8 + (lane & 7)][ks * 16 + (mat & 1) * 8]);
          mma_bf16(acc[part][2 * j2], af, b0, b1);
          mma_bf16(acc[part][2 * j2 + 1], af, b2, b3);
        }
    }
  }
  cp_async_wait<0>();
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = warp * 16 + g + 8 * half;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int c = n0 + 8 * j + 2 * t4 + e;
        if (c >= n) continue;
        float v = acc[0][j][2 * half + e];
        if (DUAL) v = gated_unit(v, acc[PARTS - 1][j][2 * half + e], alpha, limit);
        out[(size_t)(row0 + r) * n + c] = __float2bfloat16_rn(v);
      }
    }
  }
}

// ---------------------------------------------------------------------------------
// y[t] = sum over the token's choices, in their order, of weight * (the choice's row of `rows`, or the
// token's own input h[t] for an identity expert), plus row t of `extra` when given (an expert that every
// token uses). No `weight`: every choice counts once (the weights went into the experts' inputs). One
// block per token.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const T* __restrict__ h, const int* __restrict__ place,
                                   const float* __restrict__ weight, const T* __restrict__ extra, T* __restrict__ y,
                                   int hidden, int top) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool wide = hidden % VEC == 0 && ((uintptr_t)rows & 15) == 0 && ((uintptr_t)h & 15) == 0 &&
                    ((uintptr_t)y & 15) == 0 && ((uintptr_t)extra & 15) == 0;
  if (wide) {
    // Sixteen bytes of every row at a time; a choice's place and weight are read once per piece.
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
      float acc[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
      for (int k = 0; k < top; ++k) {
        const int p = place[(size_t)t * top + k];
        const float w = weight ? weight[(size_t)t * top + k] : 1.f;
        const uint4 piece = *reinterpret_cast<const uint4*>((p >= 0 ? rows + (size_t)p * hidden : h + (size_t)t * hidden) + i);
        const T* v = reinterpret_cast<const T*>(&piece);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] += weight ? w * to_f32(v[e]) : to_f32(v[e]);
      }
      if (extra) {
        const uint4 piece = *reinterpret_cast<const uint4*>(extra + (size_t)t * hidden + i);
        const T* v = reinterpret_cast<const T*>(&piece);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] += to_f32(v[e]);
      }
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = from_f32<T>(acc[e]);
      *reinterpret_cast<uint4*>(y + (size_t)t * hidden + i) = out;
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k) {
      const int p = place[(size_t)t * top + k];
      const float v = p >= 0 ? to_f32(rows[(size_t)p * hidden + i]) : to_f32(h[(size_t)t * hidden + i]);
      acc += weight ? weight[(size_t)t * top + k] * v : v;
    }
    if (extra) acc += to_f32(extra[(size_t)t * hidden + i]);
    y[(size_t)t * hidden + i] = from_f32<T>(acc);
  }
}

template <typename T, int TOK, int THREADS, int CHUNK>
int launch_route(const T* h, const float* router, const float* correction, int tokens, int outputs, int experts,
                 int hidden, int top, int sigmoid_scores, int* choice, float* weight, int* counts, size_t smem,
                 cudaStream_t stream) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(moe_route_kernel<T, TOK, THREADS, CHUNK>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch_pdl(moe_route_kernel<T, TOK, THREADS, CHUNK>, (tokens + TOK - 1) / TOK, THREADS, smem, stream, h, router, correction, tokens,
             outputs, experts, hidden, top, sigmoid_scores, choice, weight, counts);
  return OMNIA_LAUNCH_RESULT();
}

}  // namespace

extern "C" int omnia_moe_route(const void* h, const float* router, const float* correction, int tokens, int outputs,
                               int experts, int hidden, int top, int sigmoid_scores, int* choice, float* weight,
                               int* counts, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (top < 1 || top > outputs || experts < 0 || experts > outputs || outputs > 4096) return (int)cudaErrorInvalidValue;
  const int padded = (outputs + 3) / 4 * 4;
  auto bytes = [&](int tok) { return ((size_t)tok * hidden + (size_t)2 * tok * padded) * sizeof(float); };
  // Eight tokens a block where there are enough tokens to fill the GPU so and their rows fit.
  const bool many = tokens >= 8 * omnia_sm_count() && bytes(8) <= 160 * 1024;
  if (bytes(1) > 200 * 1024) return (int)cudaErrorInvalidValue;
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (many)
      return launch_route<T, 8, 256, 4>((const T*)h, router, correction, tokens, outputs, experts, hidden, top,
                                        sigmoid_scores, choice, weight, counts, bytes(8), stream);
    return launch_route<T, 1, 1024, 1>((const T*)h, router, correction, tokens, outputs, experts, hidden, top,
                                       sigmoid_scores, choice, weight, counts, bytes(1), stream);
  });
  return (int)cudaErrorInvalidValue;
}

// Routing without a router: row `ids[t]` of an integer table [vocab, top] names token t's experts
// (the entries of a row differ), each with the weight 1 / top. An entry outside the experts, or a
// token id outside the table, sets the error word's token bit and the row falls to expert 0.
__global__ void moe_route_table_kernel(const int* __restrict__ ids, const int* __restrict__ table, int tokens, int vocab,
                                       int experts, int top, int* __restrict__ choice, float* __restrict__ weight,
                                       int* __restrict__ counts, int* err) {
  pdl_wait();
  pdl_launch_dependents();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= tokens * top) return;
  const int id = ids[i / top];
  int e = id >= 0 && id < vocab ? table[(size_t)id * top + i % top] : -1;
  if (e < 0 || e >= experts) {
    atomicOr(err, OMNIA_ERR_TOKEN_ID);
    e = 0;
  }
  choice[i] = e;
  weight[i] = 1.f / (float)top;
  atomicAdd(counts + e, 1);
}

extern "C" int omnia_moe_route_table(const int* ids, const int* table, int tokens, int vocab, int experts, int top,
                                     int* choice, float* weight, int* counts, int* err, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (top < 1 || experts < 1 || vocab < 1) return (int)cudaErrorInvalidValue;
  const int pairs = tokens * top;
  launch_pdl(moe_route_table_kernel, (pairs + 255) / 256, 256, 0, stream, ids, table, tokens, vocab, experts, top, choice,
             weight, counts, err);
  return OMNIA_LAUNCH_RESULT();
}

extern "C" int omnia_moe_tile_rows() { return TILE_ROWS; }

// After `route`: the sorted order (offsets, place, source) and the list of row tiles (of at most `tile_rows`
// rows: omnia_moe_tile_rows() for this file's products, 128 for the tcgen05 kernel's grouped form).
extern "C" int omnia_moe_plan(const int* choice, int* counts, int* cursors, int* offsets, int* tiles, int* tile_count,
                              int* place, int* source, int tokens, int top, int experts, int max_tiles,
                              int tile_rows, cudaStream_t stream) {
  if (tokens == 0) return 0;
  if (experts < 1 || experts > 4096 || tile_rows < 1) return (int)cudaErrorInvalidValue;
  const int pairs = tokens * top;
  if (pairs <= 2048) {  // a small step: the plan's block places the pairs as well
    launch_pdl(moe_plan_kernel, 1, 256, (size_t)(experts + 1) * 2 * sizeof(int), stream, counts, cursors, offsets, tiles,
               tile_count, experts, max_tiles, tile_rows, choice, place, source, pairs, top);
    return OMNIA_LAUNCH_RESULT();
  }
  launch_pdl(moe_plan_kernel, 1, 256, (size_t)(experts + 1) * 2 * sizeof(int), stream, counts, cursors, offsets, tiles,
             tile_count, experts, max_tiles, tile_rows, (const int*)nullptr, (int*)nullptr, (int*)nullptr, 0, 0);
  launch_pdl(moe_scatter_kernel, (pairs + 255) / 256, 256, 0, stream, choice, (const int*)offsets, cursors, place, source,
             pairs, top, experts);
  return OMNIA_LAUNCH_RESULT();
}

// dual != 0: w holds [experts, 2 n, k] (gate rows, then up rows) and out = silu(gate) * up.
// limit > 0: the clamped unit instead, g = min(gate, limit), u = clamp(up, -limit, limit),
// out = g * sigmoid(alpha * g) * (u + 1).
extern "C" int omnia_moe_product(const void* a, const int* source, const void* w, void* out, const int* tiles,
                                 const int* tile_count, int max_tiles, int n, int k, int dual, float alpha,
                                 float limit, int dtype, int tensor_cores, cudaStream_t stream) {
  if (max_tiles == 0) return 0;
  const dim3 grid(max_tiles, (n + 63) / 64);
  if (tensor_cores) {
    if (dtype != OMNIA_BF16 || k % 8 != 0 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15)) return (int)cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(moe_product_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)tc_smem_bytes(true));
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(moe_product_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)tc_smem_bytes(false));
      if (e != cudaSuccess) return (int)e;
      configured = true;
    }
    if (dual)
      launch_pdl(moe_product_tc_kernel<true>, grid, 128, tc_smem_bytes(true), stream, (const bf16*)a, source,
                 (const bf16*)w, (bf16*)out, tiles, tile_count, n, k, alpha, limit);
    else
      launch_pdl(moe_product_tc_kernel<false>, grid, 128, tc_smem_bytes(false), stream, (const bf16*)a, source,
                 (const bf16*)w, (bf16*)out, tiles, tile_count, n, k, alpha, limit);
    return OMNIA_LAUNCH_RESULT();
  }
  OMNIA_DISPATCH_DTYPE(dtype, {
    if (dual)
      launch_pdl(moe_product_kernel<T, true>, grid, 256, 0, stream, (const T*)a, source, (const T*)w, (T*)out, tiles,
                 tile_count, n, k, alpha, limit);
    else
      launch_pdl(moe_product_kernel<T, false>, grid, 256, 0, stream, (const T*)a, source, (const T*)w, (T*)out, tiles,
                 tile_count, n, k, alpha, limit);
  });
  return OMNIA_LAUNCH_RESULT();
}

// rows[r] = h[source[r]] for the first offsets[experts] rows: the sorted order made contiguous, for a
// product that reads its operand through a tensor map.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ source, const int* __restrict__ total,
                                  T* __restrict__ rows, int hidden) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= *total) return;
  const T* src = h + (size_t)source[r] * hidden;
  T* dst = rows + (size_t)r * hidden;
  if ((hidden * sizeof(T)) % 16 == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)rows & 15) == 0) {
    const int chunks = hidden * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < chunks; i += blockDim.x)
      reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
  }
}

// rows[place[t * top + k]] = weight[t * top + k] * h[t]: the sorted order made contiguous with every
// row multiplied by its choice's weight (float32 product, rounded once), for experts that are given
// the weighted token instead of having their output weighed. Choices without a place (identity
// experts) are passed over. One block per (token, choice).
template <typename T>
__global__ void moe_weighted_rows_kernel(const T* __restrict__ h, const int* __restrict__ place,
                                         const float* __restrict__ weight, T* __restrict__ rows, int hidden, int top) {
  pdl_wait();
  pdl_launch_dependents();
  const int pair = blockIdx.x;
  const int r = place[pair];
  if (r < 0) return;
  const float w = weight[pair];
  const T* src = h + (size_t)(pair / top) * hidden;
  T* dst = rows + (size_t)r * hidden;
  constexpr int VEC = 16 / (int)sizeof(T);
  if (hidden % VEC == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)rows & 15) == 0) {
    for (int i = threadIdx.x * VEC; i < hidden; i += blockDim.x * VEC) {
      const uint4 piece = *reinterpret_cast<const uint4*>(src + i);
      const T* v = reinterpret_cast<const T*>(&piece);
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int e = 0; e < VEC; ++e) o[e] = from_f32<T>(w * to_f32(v[e]));
      *reinterpret_cast<uint4*>(dst + i) = out;
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = from_f32<T>(w * to_f32(src[i]));
}

extern "C" int omnia_moe_weighted_rows(const void* h, const int* place, const float* weight, void* rows, int pairs,
                                       int hidden, int top, int dtype, cudaStream_t stream) {
  if (pairs == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(moe_weighted_rows_kernel<T>, pairs, 128, 0, stream, (const T*)h, place, weight,
                                          (T*)rows, hidden, top)));
  return OMNIA_LAUNCH_RESULT();
}

extern "C" int omnia_moe_gather(const void* h, const int* source, const int* total, void* rows, int pairs, int hidden,
                                int dtype, cudaStream_t stream) {
  if (pairs == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(moe_gather_kernel<T>, pairs, 128, 0, stream, (const T*)h, source, total,
                                          (T*)rows, hidden)));
  return OMNIA_LAUNCH_RESULT();
}

extern "C" int omnia_moe_combine(const void* rows, const void* h, const int* place, const float* weight, const void* extra,
                                 void* y, int tokens, int hidden, int top, int dtype, cudaStream_t stream) {
  if (tokens == 0) return 0;
  OMNIA_DISPATCH_DTYPE(dtype, (launch_pdl(moe_combine_kernel<T>, tokens, 256, 0, stream, (const T*)rows, (const T*)h,
                                          place, weight, (const T*)extra, (T*)y, hidden, top)));
  return OMNIA_LAUNCH_RESULT();
}
