// Generalized delta rule: per request and head a float32 state matrix S [dim keys][dim values] runs
// through the request's tokens,
//
//     u_t = k_t / sqrt(sum(k_t^2) + 1e-6)
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T        (both first terms read S_(t-1))
//     o_t = S_t^T r_t
//
// with a decay w_t = exp(-exp(-1/2) * sigmoid(d_t + w0)) and a removal rate a_t = sigmoid(e_t + a0) per
// head and key channel.  r, k, v, e and d arrive as float32 projections of the token; everything from
// there on is float32.  A value column of S never meets another one, so four lanes share a column
// (each a quarter of its rows, kept in registers) and join their sums by shuffles.
//
// A second kernel divides every head of o by its own root mean square, multiplies by a gain vector and
// by sigmoid(gate), and rounds once.
//
// A request's result depends on its own tokens and state only: the batch, the cut of a prompt into
// portions and the slot do not change the order of a single addition.
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kDeltaLanes = 4;         // lanes that share a value column
constexpr int kDeltaMaxDim = 128;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// out[t, i] = tanh(x[t * stride + i]) in the compute dtype, i < width
template <typename T>
__global__ void tanh_rows_kernel(const float* __restrict__ x, int stride, T* __restrict__ out, int width, long long total) {
  pdl_wait();
  pdl_trigger();
  const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long t = e / width;
  const int i = (int)(e % width);
  out[e] = from_float<T>(tanhf(x[t * stride + i]));
}

// grid (requests, heads); kDeltaLanes * dim threads rounded up to whole warps.
// proj: float32 rows [r | k | v | ... ] with heads side by side inside each part; `r_off`, `k_off`, `v_off`,
// `a_off` are the first columns of r, k, v and the removal projection; `decay` is its own tensor
// [T, heads * dim] (the decay projection, before its bias).  R = rows of a lane.
template <int R>
__global__ void __launch_bounds__(kDeltaLanes * kDeltaMaxDim)
delta_scan_kernel(const float* __restrict__ proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                  const float* __restrict__ decay, int decay_stride, const float* __restrict__ decay_bias,
                  const float* __restrict__ removal_bias, float* __restrict__ out, int out_stride,
                  float* __restrict__ state, const int* __restrict__ query_start, const int* __restrict__ slots,
                  const int* __restrict__ request_active, int heads, int dim, int max_slots, int* err) {
  constexpr int kPad = kDeltaLanes * R;          // rows as the lanes see them (dim rounded up)
  __shared__ __align__(16) float w_s[2][kPad], au_s[2][kPad], u_s[2][kPad], k_s[2][kPad], r_s[2][kPad];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31;
  const int column = tid / kDeltaLanes, part = tid % kDeltaLanes;
  const bool live = column < dim;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (tid == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  float* s_base = state + ((size_t)slot * heads + head) * dim * dim;
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    s[i] = (live && row < dim) ? s_base[(size_t)row * dim + column] : 0.f;
  }
  if (tid < kPad) {
#pragma unroll
    for (int b = 0; b < 2; ++b) w_s[b][tid] = au_s[b][tid] = u_s[b][tid] = k_s[b][tid] = r_s[b][tid] = 0.f;
  }
  const int base = head * dim;
  const float w0 = tid < dim ? decay_bias[base + tid] : 0.f;
  const float a0 = tid < dim ? removal_bias[base + tid] : 0.f;
  const float decay_rate = -0.6065306597126334f;       // -exp(-1/2)
  const bool stager = tid < ((dim + 31) / 32) * 32;   // whole warps whose threads own an element i = tid

  // what token t needs from memory is asked for while token t - 1 is computed
  float kx = 0.f, rx = 0.f, ax = 0.f, dx = 0.f, vx = 0.f, ksq = 0.f;
  auto fetch = [&](int t) {
    const float* row = proj + (size_t)t * proj_stride;
    if (stager) {
      ksq = 0.f;
      for (int i = lane; i < dim; i += 32) {
        const float x = row[k_off + base + i];
        ksq = fmaf(x, x, ksq);
      }
      if (tid < dim) {
        kx = row[k_off + base + tid];
        rx = row[r_off + base + tid];
        ax = row[a_off + base + tid];
        dx = decay[(size_t)t * decay_stride + base + tid];
      }
    }
    if (live) vx = row[v_off + base + column];
  };
  if (begin < end) fetch(begin);
  for (int t = begin; t < end; ++t) {
    const int buf = (t - begin) & 1;
    if (stager) {
      const float total = warp_sum(ksq);
      if (tid < dim) {
        const float unit = kx * rsqrtf(total + 1e-6f);
        w_s[buf][tid] = expf(decay_rate * sigmoid_f(dx + w0));
        au_s[buf][tid] = sigmoid_f(ax + a0) * unit;
        u_s[buf][tid] = unit;
        k_s[buf][tid] = kx;
        r_s[buf][tid] = rx;
      }
    }
    const float v = vx;
    __syncthreads();
    if (t + 1 < end) fetch(t + 1);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) dot = fmaf(u_s[buf][part * R + i], s[i], dot);
    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      s[i] = fmaf(w_s[buf][row], s[i], fmaf(k_s[buf][row], v, -au_s[buf][row] * dot));
      o = fmaf(r_s[buf][row], s[i], o);
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    if (live && part == 0) out[(size_t)t * out_stride + base + column] = o;
    // the buffers of token t are written again for token t + 2, after the barrier of token t + 1
  }
  if (request_active[request] && live) {
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      if (row < dim) s_base[(size_t)row * dim + column] = s[i];
    }
  }
}

// out[t, g * size + i] = gain[g * size + i] * o[t, g, i] / sqrt(mean_i(o[t, g, :]^2) + eps) * sigmoid(gate[t, g * size + i])
// grid (tokens, groups), one warp.
template <typename T>
__global__ void __launch_bounds__(32)
group_gate_norm_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ gate, int gate_stride,
                       const float* __restrict__ gain, T* __restrict__ out, int out_stride, int size, float eps) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, g = blockIdx.y, lane = threadIdx.x;
  const float* row = o + (size_t)t * o_stride + (size_t)g * size;
  float sq = 0.f;
  for (int i = lane; i < size; i += 32) sq = fmaf(row[i], row[i], sq);
  const float inv = rsqrtf(warp_sum(sq) / (float)size + eps);
  for (int i = lane; i < size; i += 32) {
    const int c = g * size + i;
    const float z = gate[(size_t)t * gate_stride + c];
    out[(size_t)t * out_stride + c] = from_float<T>(gain[c] * (row[i] * inv) * sigmoid_f(z));
  }
}

}  // namespace cie

#define DISPATCH_DTYPE(code, name, ...)                              \
  if ((code) == cie::kFloat32) { using T = float; __VA_ARGS__ }      \
  else if ((code) == cie::kBFloat16) { using T = __nv_bfloat16; __VA_ARGS__ } \
  else CIE_FAIL("%s: unknown dtype code %d", name, (code));

extern "C" int cie_delta_max_dim() { return cie::kDeltaMaxDim; }

extern "C" int cie_tanh_rows(const float* x, int stride, void* out, int rows, int width, int dtype, void* stream) {
  using namespace cie;
  const long long total = (long long)rows * width;
  if (total <= 0) return 0;
  DISPATCH_DTYPE(dtype, "tanh_rows", {
    CIE_LAUNCH("tanh_rows", tanh_rows_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
               (cudaStream_t)stream, x, stride, (T*)out, width, total);
  })
  return 0;
}

extern "C" int cie_delta_scan(const float* proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                              const float* decay, int decay_stride, const float* decay_bias,
                              const float* removal_bias, float* out, int out_stride, float* state,
                              const int* query_start, const int* slots, const int* request_active, int requests,
                              int heads, int dim, int max_slots, int* err, void* stream) {
  using namespace cie;
  if (requests <= 0) return 0;
  if (dim < 1 || dim > kDeltaMaxDim) CIE_FAIL("delta_scan: head size %d is outside 1..%d", dim, kDeltaMaxDim);
  const int threads = (kDeltaLanes * dim + 31) / 32 * 32;
  const dim3 grid(requests, heads);
#define CIE_DELTA_SCAN(R)                                                                                        \
  CIE_LAUNCH("delta_scan", delta_scan_kernel<R>, grid, dim3(threads), 0, (cudaStream_t)stream, proj, proj_stride, \
             r_off, k_off, v_off, a_off, decay, decay_stride, decay_bias, removal_bias, out, out_stride, state,  \
             query_start, slots, request_active, heads, dim, max_slots, err)
  if (dim <= 32) { CIE_DELTA_SCAN(8); }
  else if (dim <= 64) { CIE_DELTA_SCAN(16); }
  else { CIE_DELTA_SCAN(32); }
#undef CIE_DELTA_SCAN
  return 0;
}

extern "C" int cie_group_gate_norm(const float* o, int o_stride, const float* gate, int gate_stride,
                                   const float* gain, void* out, int out_stride, int tokens, int groups, int size,
                                   float eps, int dtype, void* stream) {
  using namespace cie;
  if (tokens <= 0 || groups <= 0) return 0;
  if (groups > 65535) CIE_FAIL("group_gate_norm: too many groups");
  DISPATCH_DTYPE(dtype, "group_gate_norm", {
    CIE_LAUNCH("group_gate_norm", group_gate_norm_kernel<T>, dim3(tokens, groups), dim3(32), 0, (cudaStream_t)stream,
               o, o_stride, gate, gate_stride, gain, (T*)out, out_stride, size, eps);
  })
  return 0;
}
