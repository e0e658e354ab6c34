// Routed experts (mixture of experts) for a flat batch of tokens:
//
//   route      router logits in float32 (token row times a float32 router matrix), a score function
//              over all experts (softmax), the `top` largest of score + correction, and as mixing
//              weights the scores of the chosen experts (optionally renormalised to sum 1)
//   plan       counts per expert -> offsets; every (token, choice) pair gets a place in its expert's
//              run of rows; runs are cut into tiles of 64 rows for the grouped products
//   gate_up    rows gathered by place, times the expert's stacked gate and up matrices, SiLU(gate)*up
//   down       times the expert's down matrix, written to the pair's own row (float32)
//   combine    y[t] = sum over the token's choices, in the order they were chosen, of weight * row
//
// The grouped products here run on the CUDA cores with float32 accumulation, one fused multiply-add
// per k in ascending order: the 32-bit path's products, and what every shape can fall back on.  A
// pair's row does not depend on which place it got, so the batch never changes a result.
#include "common.cuh"

#include <cfloat>

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kMaxExperts = 1024;
constexpr int kRowTile = 64;          // rows of a tile of the grouped products

// ---------------------------------------------------------------- route
// One warp per token.  ids / weights: [tokens][top]; counts[e] += 1 per choice.
template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ x, const float* __restrict__ router,
                                 const float* __restrict__ correction, int* __restrict__ ids,
                                 float* __restrict__ weights, int* __restrict__ counts, int tokens,
                                 int hidden, int experts, int top, int renormalize) {
  extern __shared__ float score_s[];      // [warps][2 * experts]: scores, then choice scores
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* score = score_s + (size_t)warp * 2 * experts;
  float* choice = score + experts;
  const T* row = x + (size_t)t * hidden;
  for (int e = 0; e < experts; ++e) {
    const float* w = router + (size_t)e * hidden;
    float dot = 0.f;
    for (int k = lane; k < hidden; k += 32) dot = fmaf(to_float(row[k]), w[k], dot);
    dot = warp_sum(dot);
    if (lane == 0) score[e] = dot;
  }
  __syncwarp();
  float m = -FLT_MAX;
  for (int e = lane; e < experts; e += 32) m = fmaxf(m, score[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) sum += expf(score[e] - m);
  sum = warp_sum(sum);
  for (int e = lane; e < experts; e += 32) {
    const float s = expf(score[e] - m) / sum;
    score[e] = s;
    choice[e] = s + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  float chosen_sum = 0.f;
  for (int j = 0; j < top; ++j) {
    float best = -FLT_MAX;
    int best_e = experts;
    for (int e = lane; e < experts; e += 32)
      if (choice[e] > best) { best = choice[e]; best_e = e; }
    // largest value, lowest index on ties
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, offset);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, offset);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (lane == 0) {
      ids[(size_t)t * top + j] = best_e;
      weights[(size_t)t * top + j] = score[best_e];
      choice[best_e] = -FLT_MAX;
      atomicAdd(counts + best_e, 1);
    }
    chosen_sum += score[best_e];
    __syncwarp();
  }
  if (renormalize && lane < top) weights[(size_t)t * top + lane] /= chosen_sum;
}

// ---------------------------------------------------------------- plan
// One block.  offsets[e] = first place of expert e (offsets[experts] = pairs); place_to_pair[p] =
// the (token, choice) pair at place p; tiles: (expert, first place, rows) per tile, tile_count[0].
__global__ void moe_plan_kernel(const int* __restrict__ ids, const int* __restrict__ counts,
                                int* __restrict__ offsets, int* __restrict__ cursors,
                                int* __restrict__ place_to_pair, int* __restrict__ tiles,
                                int* __restrict__ tile_count, int pairs, int experts) {
  __shared__ int off_s[kMaxExperts + 1];
  __shared__ int tile_s[kMaxExperts + 1];
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x == 0) {
    int total = 0, tile_total = 0;
    for (int e = 0; e < experts; ++e) {
      off_s[e] = total;
      tile_s[e] = tile_total;
      total += counts[e];
      tile_total += (counts[e] + kRowTile - 1) / kRowTile;
    }
    off_s[experts] = total;
    tile_s[experts] = tile_total;
    tile_count[0] = tile_total;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) {
    offsets[e] = off_s[e];
    if (e < experts) {
      cursors[e] = 0;
      const int n = off_s[e + 1] - off_s[e];
      for (int j = 0, tile = tile_s[e]; j < n; j += kRowTile, ++tile) {
        tiles[3 * tile] = e;
        tiles[3 * tile + 1] = off_s[e] + j;
        tiles[3 * tile + 2] = min(kRowTile, n - j);
      }
    }
  }
  __syncthreads();
  for (int pair = threadIdx.x; pair < pairs; pair += blockDim.x) {
    const int e = ids[pair];
    place_to_pair[off_s[e] + atomicAdd(cursors + e, 1)] = pair;
  }
}

// ---------------------------------------------------------------- grouped products (CUDA cores)
// Tile y of the grid is tile y of the plan (blocks beyond tile_count leave at once).
//   kGateUp  A row p = x[place_to_pair[p] / top]; W = w_gate[e], w_up[e] ([ff][hidden] each);
//            out[p][n] = SiLU(a.gate_n) * (a.up_n), activation type, rows by place
//   else     A row p = act[p]; W = w_down[e] ([hidden][ff]); out[place_to_pair[p]][n], float32
template <typename T, bool kGateUp>
__global__ void __launch_bounds__(256)
moe_grouped_simt_kernel(const T* __restrict__ a, const T* __restrict__ w0, const T* __restrict__ w1,
                        void* __restrict__ out, const int* __restrict__ place_to_pair,
                        const int* __restrict__ tiles, const int* __restrict__ tile_count, int top,
                        int n_total, int k_total) {
  constexpr int kTileN = 64, kTileK = 16;
  __shared__ float a_tile[kTileK][kRowTile + 4];
  __shared__ float w_tile[kGateUp ? 2 : 1][kTileK][kTileN + 4];
  __shared__ int src_row[kRowTile];
  pdl_wait();
  pdl_trigger();
  if ((int)blockIdx.y >= tile_count[0]) return;
  const int expert = tiles[3 * blockIdx.y], place0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int tid = threadIdx.x;
  if (tid < kRowTile) {
    int r = -1;
    if (tid < rows) r = kGateUp ? place_to_pair[place0 + tid] / top : place0 + tid;
    src_row[tid] = r;
  }
  __syncthreads();
  const int n0 = blockIdx.x * kTileN;
  const T* wg = w0 + (size_t)expert * n_total * k_total;
  const T* wu = kGateUp ? w1 + (size_t)expert * n_total * k_total : nullptr;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {}, acc_up[kGateUp ? 4 : 1][4] = {};
  for (int k0 = 0; k0 < k_total; k0 += kTileK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      const int r = e / kTileK, kk = e % kTileK;
      const int gk = k0 + kk, gn = n0 + r;
      const int row = src_row[r];
      a_tile[kk][r] = (row >= 0 && gk < k_total) ? to_float(a[(size_t)row * k_total + gk]) : 0.f;
      const bool in = gn < n_total && gk < k_total;
      w_tile[0][kk][r] = in ? to_float(wg[(size_t)gn * k_total + gk]) : 0.f;
      if constexpr (kGateUp) w_tile[1][kk][r] = in ? to_float(wu[(size_t)gn * k_total + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < kTileK; ++kk) {
      float av[4], wv[4], uv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = a_tile[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        wv[j] = w_tile[0][kk][tn + j];
        if constexpr (kGateUp) uv[j] = w_tile[1][kk][tn + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if constexpr (kGateUp) acc_up[i][j] = fmaf(av[i], uv[j], acc_up[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = tm + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= n_total) continue;
      if constexpr (kGateUp) {
        const float g = acc[i][j];
        reinterpret_cast<T*>(out)[(size_t)(place0 + r) * n_total + gn] =
            from_float<T>(g / (1.f + expf(-g)) * acc_up[i][j]);
      } else {
        reinterpret_cast<float*>(out)[(size_t)place_to_pair[place0 + r] * n_total + gn] = acc[i][j];
      }
    }
  }
}

// y[t][i] = sum_j weights[t][j] * rows[t * top + j][i], j ascending; float32 or activation type out.
template <typename TOut>
__global__ void moe_combine_kernel(const float* __restrict__ rows, const float* __restrict__ weights,
                                   TOut* __restrict__ y, int hidden, int top) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < top; ++j)
      total = fmaf(weights[(size_t)t * top + j], rows[((size_t)t * top + j) * hidden + i], total);
    y[(size_t)t * hidden + i] = from_float<TOut>(total);
  }
}

}  // namespace cie

using namespace cie;

extern "C" int cie_moe_row_tile() { return kRowTile; }

// counts, offsets (experts + 1), cursors, tile_count (1) and tiles (3 * (pairs / 64 + experts)) are
// int32 scratch of the caller; counts is zeroed here.
extern "C" int cie_moe_route(const void* x, const float* router, const float* correction, int* ids,
                             float* weights, int* counts, int* offsets, int* cursors, int* place_to_pair,
                             int* tiles, int* tile_count, int tokens, int hidden, int experts, int top,
                             int renormalize, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  if (experts < 1 || experts > kMaxExperts) CIE_FAIL("moe_route: 1..%d experts, got %d", kMaxExperts, experts);
  if (top < 1 || top > experts || top > 32) CIE_FAIL("moe_route: top %d of %d experts (at most 32)", top, experts);
  cudaStream_t s = (cudaStream_t)stream;
  if (cudaMemsetAsync(counts, 0, sizeof(int) * experts, s) != cudaSuccess) CIE_FAIL("moe_route: memset failed");
  const int warps = 4;
  const size_t smem = (size_t)warps * 2 * experts * sizeof(float);
  const int blocks = (tokens + warps - 1) / warps;
  if (dtype == kFloat32) {
    CIE_LAUNCH("moe_route", moe_route_kernel<float>, dim3(blocks), dim3(warps * 32), smem, s, (const float*)x, router,
               correction, ids, weights, counts, tokens, hidden, experts, top, renormalize);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("moe_route", moe_route_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), smem, s,
               (const __nv_bfloat16*)x, router, correction, ids, weights, counts, tokens, hidden, experts, top,
               renormalize);
  } else {
    CIE_FAIL("moe_route: unknown element type code %d", dtype);
  }
  CIE_LAUNCH("moe_plan", moe_plan_kernel, dim3(1), dim3(1024), 0, s, ids, counts, offsets, cursors, place_to_pair,
             tiles, tile_count, tokens * top, experts);
  return 0;
}

// act: [pairs][ff] activation type, rows by place.  w_gate, w_up: [experts][ff][hidden].
extern "C" int cie_moe_gate_up_simt(const void* x, const void* w_gate, const void* w_up, void* act,
                                    const int* place_to_pair, const int* tiles, const int* tile_count,
                                    int tokens, int top, int experts, int ff, int hidden, int dtype,
                                    void* stream) {
  if (tokens <= 0) return 0;
  const int max_tiles = (tokens * top + kRowTile - 1) / kRowTile + experts;
  dim3 grid((ff + 63) / 64, max_tiles);
  if (dtype == kFloat32) {
    CIE_LAUNCH("moe_gate_up", (moe_grouped_simt_kernel<float, true>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const float*)x, (const float*)w_gate, (const float*)w_up, act, place_to_pair, tiles, tile_count, top,
               ff, hidden);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("moe_gate_up", (moe_grouped_simt_kernel<__nv_bfloat16, true>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate, (const __nv_bfloat16*)w_up, act, place_to_pair,
               tiles, tile_count, top, ff, hidden);
  } else {
    CIE_FAIL("moe_gate_up: unknown element type code %d", dtype);
  }
  return 0;
}

// rows: float32 [pairs][hidden], row of pair (t, j) at t * top + j.  w_down: [experts][hidden][ff].
extern "C" int cie_moe_down_simt(const void* act, const void* w_down, float* rows, const int* place_to_pair,
                                 const int* tiles, const int* tile_count, int tokens, int top, int experts,
                                 int ff, int hidden, int dtype, void* stream) {
  if (tokens <= 0) return 0;
  const int max_tiles = (tokens * top + kRowTile - 1) / kRowTile + experts;
  dim3 grid((hidden + 63) / 64, max_tiles);
  if (dtype == kFloat32) {
    CIE_LAUNCH("moe_down", (moe_grouped_simt_kernel<float, false>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const float*)act, (const float*)w_down, (const float*)nullptr, (void*)rows, place_to_pair, tiles,
               tile_count, top, hidden, ff);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("moe_down", (moe_grouped_simt_kernel<__nv_bfloat16, false>), grid, dim3(256), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, (const __nv_bfloat16*)nullptr, (void*)rows,
               place_to_pair, tiles, tile_count, top, hidden, ff);
  } else {
    CIE_FAIL("moe_down: unknown element type code %d", dtype);
  }
  return 0;
}

// y: [tokens][hidden], float32 (out_dtype 0) or bfloat16 (1).
extern "C" int cie_moe_combine(const float* rows, const float* weights, void* y, int tokens, int hidden,
                               int top, int out_dtype, void* stream) {
  if (tokens <= 0) return 0;
  int threads = 32;
  while (threads < hidden / 4 && threads < 1024) threads <<= 1;
  if (out_dtype == kFloat32) {
    CIE_LAUNCH("moe_combine", moe_combine_kernel<float>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream, rows,
               weights, (float*)y, hidden, top);
  } else if (out_dtype == kBFloat16) {
    CIE_LAUNCH("moe_combine", moe_combine_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, (cudaStream_t)stream,
               rows, weights, (__nv_bfloat16*)y, hidden, top);
  } else {
    CIE_FAIL("moe_combine: unknown element type code %d", out_dtype);
  }
  return 0;
}
