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
