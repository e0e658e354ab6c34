// Linear attention with a fixed decay per head ("lightning attention"), as the recurrence
//
//     S_t = decay_h * S_(t-1) + k_t v_t^T          (S: [dim][vdim], float32, one per request and head)
//     o_t = S_t^T q_t
//
// over a ragged batch: every request brings one or more new tokens and continues from the state its
// slot holds.  q, k and v arrive as one projected row per token, [q | k | v | gate] with heads side
// by side inside each part, still without their activation: SiLU is applied here in float32, and
// everything that enters the recurrence stays float32.  A second kernel normalises the
// concatenated heads of o (RMS, gain vector), multiplies by sigmoid(gate) and rounds once.
//
// A request's result depends on its own tokens and state only: the batch, the cut of a prompt into
// portions and the slot do not change the order of a single addition.
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kScanWarps = 8;        // warps of a scan block; warp w owns state rows w, w + 8, ...
constexpr int kScanColumns = 32;     // value columns of a block: one per lane
constexpr int kScanRows = 32;        // state rows a warp keeps in registers (dim <= 8 * 32)

__device__ __forceinline__ float silu_f(float z) { return z / (1.f + expf(-z)); }

// grid: (requests, heads, ceil(vdim / 32)).
template <typename T>
__global__ void __launch_bounds__(kScanWarps * 32)
lightning_scan_kernel(const T* __restrict__ proj, int proj_stride, float* __restrict__ out, int out_stride,
                      float* __restrict__ state, const float* __restrict__ decay,
                      const int* __restrict__ query_start, const int* __restrict__ slots,
                      const int* __restrict__ request_active, int heads, int dim, int vdim, int max_slots,
                      int* err) {
  __shared__ float q_s[2][kScanWarps * kScanRows], k_s[2][kScanWarps * kScanRows];
  __shared__ float part_s[2][kScanWarps][kScanColumns];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int column = blockIdx.z * kScanColumns + lane;
  const bool live = column < vdim;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (threadIdx.x == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  const float d = decay[head];
  float* s_base = state + (((size_t)slot * heads + head) * dim) * vdim;
  float s[kScanRows];
#pragma unroll
  for (int r = 0; r < kScanRows; ++r) {
    const int i = warp + kScanWarps * r;
    s[r] = (i < dim && live) ? s_base[(size_t)i * vdim + column] : 0.f;
  }
  const int q_off = head * dim, k_off = heads * dim + head * dim, v_off = 2 * heads * dim + head * vdim;
  for (int t = begin; t < end; ++t) {
    const int buf = (t - begin) & 1;
    const T* row = proj + (size_t)t * proj_stride;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      q_s[buf][i] = silu_f(to_float(row[q_off + i]));
      k_s[buf][i] = silu_f(to_float(row[k_off + i]));
    }
    const float v = live ? silu_f(to_float(row[v_off + column])) : 0.f;
    __syncthreads();
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < kScanRows; ++r) {
      const int i = warp + kScanWarps * r;
      if (i < dim) {
        s[r] = fmaf(d, s[r], k_s[buf][i] * v);
        o = fmaf(s[r], q_s[buf][i], o);
      }
    }
    part_s[buf][warp][lane] = o;
    __syncthreads();
    if (warp == 0 && live) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kScanWarps; ++w) total += part_s[buf][w][lane];
      out[(size_t)t * out_stride + head * vdim + column] = total;
    }
    // the buffers of token t are read again only after the first barrier of token t + 2
  }
  if (request_active[request] && live) {
#pragma unroll
    for (int r = 0; r < kScanRows; ++r) {
      const int i = warp + kScanWarps * r;
      if (i < dim) s_base[(size_t)i * vdim + column] = s[r];
    }
  }
}

// ---------------------------------------------------------------- prompt portions in chunks
// The same recurrence over chunks of up to kChunk tokens, so that a long portion is work for many
// CTAs instead of one chain (all float32, CUDA cores; key and value sizes up to 128):
//   1. per (chunk, head):    U = sum_j decay^(n-1-j) k_j v_j^T                       (n tokens in the chunk)
//   2. per (request, head):  walks its chunks in order, S <- decay^n S + U, leaving in U's place the
//                            state BEFORE the chunk; the last S goes back to the slot
//   3. per (chunk, head):    o_i = decay^(i+1) S_before^T q_i + sum_{j<=i} decay^(i-j) (q_i.k_j) v_j
// Chunks come as a work list (request, first token row, tokens) made on the host from the step's
// portion lengths; a request's chunks follow each other.
constexpr int kChunk = 32;
constexpr int kChunkDim = 128;       // largest key and value size of the chunked kernels
constexpr int kChunkRows = kChunkDim / kScanWarps;      // state rows of a warp
constexpr int kChunkCols = kChunkDim / 32;              // value columns of a lane

__device__ __forceinline__ float decay_power(float log2_decay, int n) { return n == 0 ? 1.f : exp2f(log2_decay * (float)n); }

template <typename T> struct Piece;                 // a 16-byte piece of a row
template <> struct Piece<float> { static constexpr int n = 4; };
template <> struct Piece<__nv_bfloat16> { static constexpr int n = 8; };

// dst[j * ld + i] = SiLU(proj[row0 + j][col0 + i]) * factor(j) for j < n, i < width: 16-byte loads where
// the columns allow (one index division per piece instead of per element), else element by element.
template <typename T, typename Factor>
__device__ __forceinline__ void stage_silu(float* __restrict__ dst, int ld, const T* __restrict__ proj, int proj_stride,
                                           int row0, int n, int col0, int width, Factor factor) {
  constexpr int V = Piece<T>::n;
  if (width % V == 0 && col0 % V == 0 && proj_stride % V == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0) {
    const int pieces = width / V;
    for (int e = threadIdx.x; e < n * pieces; e += blockDim.x) {
      const int j = e / pieces, i = (e % pieces) * V;
      const uint4 raw = *reinterpret_cast<const uint4*>(proj + (size_t)(row0 + j) * proj_stride + col0 + i);
      const T* v = reinterpret_cast<const T*>(&raw);
      const float f = factor(j);
#pragma unroll
      for (int x = 0; x < V; ++x) dst[j * ld + i + x] = silu_f(to_float(v[x])) * f;
    }
    return;
  }
  for (int e = threadIdx.x; e < n * width; e += blockDim.x) {
    const int j = e / width, i = e % width;
    dst[j * ld + i] = silu_f(to_float(proj[(size_t)(row0 + j) * proj_stride + col0 + i])) * factor(j);
  }
}

template <typename T>
__global__ void __launch_bounds__(kScanWarps * 32)
lightning_chunk_state_kernel(const T* __restrict__ proj, int proj_stride, float* __restrict__ chunk_state,
                             const float* __restrict__ decay, const int* __restrict__ chunk_row,
                             const int* __restrict__ chunk_count, int heads, int dim, int vdim) {
  extern __shared__ __align__(16) float smem[];
  float* k_s = smem;                          // [kChunk][dim], times decay^(n-1-j)
  float* v_s = smem + kChunk * dim;           // [kChunk][vdim]
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  const float log2_d = log2f(decay[head]);
  const int k_off = heads * dim + head * dim, v_off = 2 * heads * dim + head * vdim;
  stage_silu(k_s, dim, proj, proj_stride, row0, n, k_off, dim, [&](int j) { return decay_power(log2_d, n - 1 - j); });
  stage_silu(v_s, vdim, proj, proj_stride, row0, n, v_off, vdim, [](int) { return 1.f; });
  __syncthreads();
  // a warp owns kChunkRows state rows that follow each other (its k values come as 16-byte loads), a
  // lane the value columns lane, lane + 32, ...
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = warp * kChunkRows;
  const bool whole = dim % 4 == 0 && i0 + kChunkRows <= dim;
  float u[kChunkRows][kChunkCols] = {};
  for (int j = 0; j < n; ++j) {
    float vv[kChunkCols], kv[kChunkRows];
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c) vv[c] = lane + 32 * c < vdim ? v_s[j * vdim + lane + 32 * c] : 0.f;
    if (whole) {
#pragma unroll
      for (int r = 0; r < kChunkRows; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + j * dim + i0 + r);
        kv[r] = k4.x; kv[r + 1] = k4.y; kv[r + 2] = k4.z; kv[r + 3] = k4.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < kChunkRows; ++r) kv[r] = i0 + r < dim ? k_s[j * dim + i0 + r] : 0.f;
    }
#pragma unroll
    for (int r = 0; r < kChunkRows; ++r)
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) u[r][c] = fmaf(kv[r], vv[c], u[r][c]);
  }
  float* dst = chunk_state + ((size_t)chunk * heads + head) * dim * vdim;
#pragma unroll
  for (int r = 0; r < kChunkRows; ++r) {
    const int i = i0 + r;
    if (i >= dim) continue;
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c)
      if (lane + 32 * c < vdim) dst[(size_t)i * vdim + lane + 32 * c] = u[r][c];
  }
}

// grid: (requests, heads, blocks over dim * vdim)
__global__ void lightning_chunk_prefix_kernel(float* __restrict__ chunk_state, float* __restrict__ state,
                                              const float* __restrict__ decay,
                                              const int* __restrict__ request_chunk_start,
                                              const int* __restrict__ chunk_count, const int* __restrict__ slots,
                                              const int* __restrict__ request_active, int heads, int dim, int vdim,
                                              int max_slots, int* err) {
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= dim * vdim) return;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (e == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const float log2_d = log2f(decay[head]);
  float* cell = state + ((size_t)slot * heads + head) * dim * vdim + e;
  float s = *cell;
  const size_t stride = (size_t)heads * dim * vdim;
  const int last = request_chunk_start[request + 1];
  // eight chunks at a time: their sums are asked for together, before the first store, so that the
  // walk waits for memory once per eight chunks and not once per chunk
  constexpr int kBatch = 8;
  for (int chunk = request_chunk_start[request]; chunk < last; chunk += kBatch) {
    float* u = chunk_state + ((size_t)chunk * heads + head) * dim * vdim + e;
    float gained[kBatch], power[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const bool in = chunk + b < last;
      gained[b] = in ? u[b * stride] : 0.f;
      power[b] = in ? decay_power(log2_d, chunk_count[chunk + b]) : 1.f;
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (chunk + b < last) {
        u[b * stride] = s;
        s = fmaf(power[b], s, gained[b]);
      }
    }
  }
  if (request_active[request]) *cell = s;
}

template <typename T>
__global__ void __launch_bounds__(kScanWarps * 32)
lightning_chunk_output_kernel(const T* __restrict__ proj, int proj_stride, float* __restrict__ out, int out_stride,
                              const float* __restrict__ chunk_state, const float* __restrict__ decay,
                              const int* __restrict__ chunk_row, const int* __restrict__ chunk_count, int heads,
                              int dim, int vdim) {
  extern __shared__ __align__(16) float smem[];
  float* q_s = smem;                              // [kChunk][dim]
  float* k_s = q_s + kChunk * dim;                // [kChunk][dim + 1]
  float* v_s = k_s + kChunk * (dim + 1);          // [kChunk][vdim]
  float* a_s = v_s + kChunk * vdim;               // [kChunk][kChunk]
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  const float log2_d = log2f(decay[head]);
  const int q_off = head * dim, k_off = heads * dim + head * dim, v_off = 2 * heads * dim + head * vdim;
  stage_silu(q_s, dim, proj, proj_stride, row0, n, q_off, dim, [](int) { return 1.f; });
  stage_silu(k_s, dim + 1, proj, proj_stride, row0, n, k_off, dim, [](int) { return 1.f; });
  stage_silu(v_s, vdim, proj, proj_stride, row0, n, v_off, vdim, [](int) { return 1.f; });
  __syncthreads();
  // a[i][j] = decay^(i-j) q_i.k_j for j <= i (lanes run over j: k rows are padded by one element)
  for (int e = threadIdx.x; e < n * kChunk; e += blockDim.x) {
    const int i = e / kChunk, j = e % kChunk;
    float dot = 0.f;
    if (j <= i) {
      for (int x = 0; x < dim; ++x) dot = fmaf(q_s[i * dim + x], k_s[j * (dim + 1) + x], dot);
      dot *= decay_power(log2_d, i - j);
    }
    a_s[e] = dot;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* before = chunk_state + ((size_t)chunk * heads + head) * dim * vdim;
  // a warp takes tokens warp, warp + 8, ...; a lane the value columns lane, lane + 32, ...
  constexpr int kTokens = kChunk / kScanWarps;
  float inter[kTokens][kChunkCols] = {}, intra[kTokens][kChunkCols] = {};
  const int dim4 = dim % 4 == 0 ? dim : 0;       // four state rows a step where the q rows allow 16-byte loads
  for (int x = 0; x < dim4; x += 4) {
    float sv[4][kChunkCols];
#pragma unroll
    for (int y = 0; y < 4; ++y)
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) sv[y][c] = lane + 32 * c < vdim ? before[(size_t)(x + y) * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kScanWarps * t;
      const float4 q4 = i < n ? *reinterpret_cast<const float4*>(q_s + i * dim + x) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) {
        inter[t][c] = fmaf(q4.x, sv[0][c], inter[t][c]);
        inter[t][c] = fmaf(q4.y, sv[1][c], inter[t][c]);
        inter[t][c] = fmaf(q4.z, sv[2][c], inter[t][c]);
        inter[t][c] = fmaf(q4.w, sv[3][c], inter[t][c]);
      }
    }
  }
  for (int x = dim4; x < dim; ++x) {
    float sv[kChunkCols];
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c) sv[c] = lane + 32 * c < vdim ? before[(size_t)x * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kScanWarps * t;
      const float qv = i < n ? q_s[i * dim + x] : 0.f;
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) inter[t][c] = fmaf(qv, sv[c], inter[t][c]);
    }
  }
  for (int j = 0; j < n; ++j) {
    float vv[kChunkCols];
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c) vv[c] = lane + 32 * c < vdim ? v_s[j * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kScanWarps * t;
      const float av = (i < n && j <= i) ? a_s[i * kChunk + j] : 0.f;
#pragma unroll
      for (int c = 0; c < kChunkCols; ++c) intra[t][c] = fmaf(av, vv[c], intra[t][c]);
    }
  }
#pragma unroll
  for (int t = 0; t < kTokens; ++t) {
    const int i = warp + kScanWarps * t;
    if (i >= n) continue;
    const float carried = decay_power(log2_d, i + 1);
#pragma unroll
    for (int c = 0; c < kChunkCols; ++c)
      if (lane + 32 * c < vdim)
        out[(size_t)(row0 + i) * out_stride + head * vdim + lane + 32 * c] = fmaf(carried, inter[t][c], intra[t][c]);
  }
}

// out[t][i] = gain[i] * o[t][i] * rsqrt(mean_i(o[t]^2) + eps) * sigmoid(gate[t][i]); one block per token.
template <typename T>
__global__ void lightning_gate_norm_kernel(const float* __restrict__ o, int o_stride, const T* __restrict__ gate,
                                           int gate_stride, const float* __restrict__ gain, T* __restrict__ out,
                                           int width, float eps) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const float* row = o + (size_t)t * o_stride;
  float sq = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sq = fmaf(row[i], row[i], sq);
  const float inv = rsqrtf(block_sum(sq, scratch) / (float)width + eps);
  const T* g = gate + (size_t)t * gate_stride;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float z = to_float(g[i]);
    out[(size_t)t * width + i] = from_float<T>(gain[i] * (row[i] * inv) * (1.f / (1.f + expf(-z))));
  }
}

}  // namespace cie

using namespace cie;

// proj: [tokens][proj_stride] = [q: heads*dim | k: heads*dim | v: heads*vdim | ...]; out: float32
// [tokens][out_stride], head h at column h*vdim; state: float32 [max_slots][heads][dim][vdim].
extern "C" int cie_lightning_scan(const void* proj, int proj_stride, float* out, int out_stride, float* state,
                                  const float* decay, const int* query_start, const int* slots,
                                  const int* request_active, int requests, int heads, int dim, int vdim,
                                  int max_slots, int dtype, int* err, void* stream) {
  if (requests <= 0) return 0;
  if (dim < 1 || dim > kScanWarps * kScanRows) CIE_FAIL("lightning_scan: key size %d is outside 1..%d", dim, kScanWarps * kScanRows);
  if (vdim < 1 || heads < 1) CIE_FAIL("lightning_scan: %d heads of value size %d", heads, vdim);
  dim3 grid(requests, heads, (vdim + kScanColumns - 1) / kScanColumns);
  if (dtype == kFloat32) {
    CIE_LAUNCH("lightning_scan", lightning_scan_kernel<float>, grid, dim3(kScanWarps * 32), 0, (cudaStream_t)stream,
               (const float*)proj, proj_stride, out, out_stride, state, decay, query_start, slots, request_active,
               heads, dim, vdim, max_slots, err);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("lightning_scan", lightning_scan_kernel<__nv_bfloat16>, grid, dim3(kScanWarps * 32), 0, (cudaStream_t)stream,
               (const __nv_bfloat16*)proj, proj_stride, out, out_stride, state, decay, query_start, slots,
               request_active, heads, dim, vdim, max_slots, err);
  } else {
    CIE_FAIL("lightning_scan: unknown element type code %d", dtype);
  }
  return 0;
}

extern "C" int cie_lightning_chunk_tokens() { return kChunk; }

// The chunked form (see above).  chunk_state: float32 scratch [chunks][heads][dim][vdim].
extern "C" int cie_lightning_chunked(const void* proj, int proj_stride, float* out, int out_stride, float* state,
                                     float* chunk_state, const float* decay, const int* chunk_row,
                                     const int* chunk_count, const int* request_chunk_start, const int* slots,
                                     const int* request_active, int chunks, int requests, int heads, int dim,
                                     int vdim, int max_slots, int dtype, int* err, void* stream) {
  if (chunks <= 0 || requests <= 0) return 0;
  if (dim < 1 || dim > kChunkDim || vdim < 1 || vdim > kChunkDim)
    CIE_FAIL("lightning_chunked: key / value sizes %d / %d are outside 1..%d", dim, vdim, kChunkDim);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem1 = (size_t)kChunk * (dim + vdim) * sizeof(float);
  const size_t smem3 = (size_t)kChunk * (2 * dim + 1 + vdim + kChunk) * sizeof(float);
  dim3 grid(chunks, heads), block(kScanWarps * 32);
  dim3 grid2(requests, heads, (dim * vdim + 255) / 256);
#define CIE_CHUNKED(T)                                                                                        \
  do {                                                                                                        \
    if (smem3 > 48 * 1024 &&                                                                                  \
        cudaFuncSetAttribute(lightning_chunk_output_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                             (int)smem3) != cudaSuccess)                                                      \
      CIE_FAIL("lightning_chunked: cannot reserve %zu bytes of shared memory", smem3);                        \
    CIE_LAUNCH("lightning_chunk_state", lightning_chunk_state_kernel<T>, grid, block, smem1, s, (const T*)proj,  \
               proj_stride, chunk_state, decay, chunk_row, chunk_count, heads, dim, vdim);                    \
    CIE_LAUNCH("lightning_chunk_prefix", lightning_chunk_prefix_kernel, grid2, dim3(256), 0, s, chunk_state,   \
               state, decay, request_chunk_start, chunk_count, slots, request_active, heads, dim, vdim,       \
               max_slots, err);                                                                               \
    CIE_LAUNCH("lightning_chunk_output", lightning_chunk_output_kernel<T>, grid, block, smem3, s,              \
               (const T*)proj, proj_stride, out, out_stride, (const float*)chunk_state, decay, chunk_row,     \
               chunk_count, heads, dim, vdim);                                                                \
  } while (0)
  if (dtype == kFloat32) CIE_CHUNKED(float);
  else if (dtype == kBFloat16) CIE_CHUNKED(__nv_bfloat16);
  else CIE_FAIL("lightning_chunked: unknown element type code %d", dtype);
#undef CIE_CHUNKED
  return 0;
}

extern "C" int cie_lightning_gate_norm(const float* o, int o_stride, const void* gate, int gate_stride,
                                       const float* gain, void* out, int tokens, int width, float eps,
                                       int dtype, void* stream) {
  if (tokens <= 0) return 0;
  int threads = 32;
  while (threads < width / 4 && threads < 1024) threads <<= 1;
  if (dtype == kFloat32) {
    CIE_LAUNCH("lightning_gate_norm", lightning_gate_norm_kernel<float>, dim3(tokens), dim3(threads), 0,
               (cudaStream_t)stream, o, o_stride, (const float*)gate, gate_stride, gain, (float*)out, width, eps);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("lightning_gate_norm", lightning_gate_norm_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0,
               (cudaStream_t)stream, o, o_stride, (const __nv_bfloat16*)gate, gate_stride, gain,
               (__nv_bfloat16*)out, width, eps);
  } else {
    CIE_FAIL("lightning_gate_norm: unknown element type code %d", dtype);
  }
  return 0;
}
