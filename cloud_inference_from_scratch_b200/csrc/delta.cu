// Generalized delta rule: per request and head a float32 state matrix S [dim keys][dim values] runs
// through the request's tokens,
//
//     u_t = k_t / sqrt(sum(k_t^2) + 1e-6)
//     S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T        (both first terms read S_(t-1))
//     o_t = S_t^T r_t
//
// with a decay w_t = exp(-exp(-1/2) * sigmoid(d_t + w0)) and a removal rate a_t = sigmoid(e_t + a0) per
// head and key channel.  r, k, v, e and d arrive as float32 projections of the token; everything from
// there on is float32.  A value column of S never meets another one, so eight lanes share a column
// (each an eighth of its rows, kept in registers) and join their sums by shuffles: what bounds the
// recurrence is the chain of dependent steps of one token, and more lanes a column shorten it.
//
// A second kernel divides every head of o by its own root mean square, multiplies by a gain vector and
// by sigmoid(gate), and rounds once.
//
// A request's result depends on its own tokens and state only: the batch, the cut of a prompt into
// portions and the slot do not change the order of a single addition.
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kDeltaLanes = 8;         // lanes that share a value column
constexpr int kDeltaMaxDim = 256;       // largest head of the scan kernel
constexpr int kDeltaBlockColumns = 128;  // value columns of a block (heads above that take several blocks)
constexpr int kDeltaStreamMaxDim = 128; // largest head of the stream kernel (a column's rows are one thread's registers)

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

// grid (requests, heads, blocks of kDeltaBlockColumns value columns); kDeltaLanes threads a column, rounded up
// to whole warps.  Every block stages all rows of k, r and the rates; it keeps only its own columns of S.
// proj: float32 rows [r | k | v | ... ] with heads side by side inside each part; `r_off`, `k_off`, `v_off`,
// `a_off` are the first columns of r, k, v and the removal projection; `decay` is its own tensor
// [T, heads * dim] (the decay projection, before its bias).  R = rows of a lane.
template <int R>
__global__ void __launch_bounds__(kDeltaLanes * kDeltaBlockColumns)
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
  const int column = blockIdx.z * kDeltaBlockColumns + tid / kDeltaLanes, part = tid % kDeltaLanes;
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
  for (int i = tid; i < kPad; i += blockDim.x) {
#pragma unroll
    for (int b = 0; b < 2; ++b) w_s[b][i] = au_s[b][i] = u_s[b][i] = k_s[b][i] = r_s[b][i] = 0.f;
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
    dot += __shfl_xor_sync(0xffffffffu, dot, 4);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      s[i] = fmaf(w_s[buf][row], s[i], fmaf(k_s[buf][row], v, -au_s[buf][row] * dot));
      o = fmaf(r_s[buf][row], s[i], o);
    }
    o += __shfl_xor_sync(0xffffffffu, o, 1);
    o += __shfl_xor_sync(0xffffffffu, o, 2);
    o += __shfl_xor_sync(0xffffffffu, o, 4);
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

// ---------------------------------------------------------------- prompt portions: prepare, then stream
// For many tokens a request the scan above waits, token after token, for its own loads and for the
// exponentials of the rates.  Two kernels instead: `delta_prepare` computes, for all tokens at once,
// what the recurrence reads (w, a * u, u, k, r, v per head, float32, each padded with zeros to the rows
// the lanes keep) and `delta_stream` walks a request's tokens reading those rows through a ring of
// cp.async stages, several tokens ahead.  The arithmetic is that of the scan; the sums over a column's
// rows are added in another order (four chains a thread instead of a chain a lane).
constexpr int kDeltaStages = 3;      // stages of the ring
constexpr int kDeltaChunk = 4;       // tokens of a stage: the block meets once a stage, not once a token
constexpr int kDeltaFields = 6;      // w, a * u, u, k, r, v

// grid (tokens, heads), one warp or more; `pad` = rows as the stream kernel's lanes see them.
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const float* __restrict__ proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                     const float* __restrict__ decay, int decay_stride, const float* __restrict__ decay_bias,
                     const float* __restrict__ removal_bias, float* __restrict__ packed, int tokens, int heads, int dim,
                     int pad) {
  __shared__ float scratch[33];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, head = blockIdx.y, base = head * dim;
  const float* row = proj + (size_t)t * proj_stride;
  float sq = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {     // the order of the scan: lane l adds l, l + 32, ...
    const float x = row[k_off + base + i];
    sq = fmaf(x, x, sq);
  }
  // the scan adds a warp's 32 partial sums; here a block of one warp does the same
  const float total = block_sum(sq, scratch);
  const float inv = rsqrtf(total + 1e-6f);
  float* dst = packed + ((size_t)head * tokens + t) * kDeltaFields * pad;     // head-major: a head's tokens follow each other
  for (int i = threadIdx.x; i < pad; i += blockDim.x) {
    float w = 0.f, au = 0.f, u = 0.f, k = 0.f, r = 0.f, v = 0.f;
    if (i < dim) {
      k = row[k_off + base + i];
      r = row[r_off + base + i];
      v = row[v_off + base + i];
      u = k * inv;
      au = sigmoid_f(row[a_off + base + i] + removal_bias[base + i]) * u;
      w = expf(-0.6065306597126334f * sigmoid_f(decay[(size_t)t * decay_stride + base + i] + decay_bias[base + i]));
    }
    dst[i] = w;
    dst[pad + i] = au;
    dst[2 * pad + i] = u;
    dst[3 * pad + i] = k;
    dst[4 * pad + i] = r;
    dst[5 * pad + i] = v;
  }
}

__device__ __forceinline__ void delta_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// One thread a value column with ALL its rows in registers: every read of a token's row is then the
// same address for the whole warp (one shared-memory wavefront a load, where lanes that share a column
// read eight different places), and no sum crosses lanes.  P = rows as padded (32, 64 or 128).
template <int P>
__global__ void __launch_bounds__(kDeltaStreamMaxDim)
delta_stream_kernel(const float* __restrict__ packed, float* __restrict__ out, int out_stride, float* __restrict__ state,
                    const int* __restrict__ query_start, const int* __restrict__ slots,
                    const int* __restrict__ request_active, int tokens, int heads, int dim, int max_slots, int* err) {
  constexpr int kRow = kDeltaFields * P;             // floats of one token and head
  __shared__ __align__(16) float ring[kDeltaStages][kDeltaChunk * kRow];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int tid = threadIdx.x;
  const int column = tid;
  const bool live = column < dim;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (tid == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  float* s_base = state + ((size_t)slot * heads + head) * dim * dim;
  float s[P];
#pragma unroll
  for (int i = 0; i < P; ++i) s[i] = (live && i < dim) ? s_base[(size_t)i * dim + column] : 0.f;
  const float* rows = packed + (size_t)head * tokens * kRow;
  auto issue = [&](int chunk) {
    const int first = begin + chunk * kDeltaChunk;
    if (first < end) {
      const int count = min(kDeltaChunk, end - first) * (kRow / 4);
      const float* src = rows + (size_t)first * kRow;
      float* dst = ring[chunk % kDeltaStages];
      for (int c = tid; c < count; c += blockDim.x) delta_cp_async16(dst + 4 * c, src + 4 * c);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  for (int i = 0; i < kDeltaStages - 1; ++i) issue(i);
  const int base = head * dim;
  for (int t = begin; t < end; ++t) {
    const int chunk = (t - begin) / kDeltaChunk, place = (t - begin) % kDeltaChunk;
    if (place == 0) {
      asm volatile("cp.async.wait_group %0;\n" ::"n"(kDeltaStages - 2));
      __syncthreads();          // the chunk has landed; everybody is done with the chunk before, whose stage is filled next
      issue(chunk + kDeltaStages - 1);
    }
    const float* stage = ring[chunk % kDeltaStages] + place * kRow;
    const float4* w4 = reinterpret_cast<const float4*>(stage);
    const float4* au4 = reinterpret_cast<const float4*>(stage + P);
    const float4* u4 = reinterpret_cast<const float4*>(stage + 2 * P);
    const float4* k4 = reinterpret_cast<const float4*>(stage + 3 * P);
    const float4* r4 = reinterpret_cast<const float4*>(stage + 4 * P);
    const float v = stage[5 * P + (live ? column : 0)];
    float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;      // four chains, joined as (d0 + d1) + (d2 + d3)
#pragma unroll
    for (int i = 0; i < P / 4; ++i) {
      const float4 u = u4[i];
      d0 = fmaf(u.x, s[4 * i], d0);
      d1 = fmaf(u.y, s[4 * i + 1], d1);
      d2 = fmaf(u.z, s[4 * i + 2], d2);
      d3 = fmaf(u.w, s[4 * i + 3], d3);
    }
    const float dot = (d0 + d1) + (d2 + d3);
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int i = 0; i < P / 4; ++i) {
      const float4 w = w4[i], au = au4[i], k = k4[i], r = r4[i];
      s[4 * i] = fmaf(w.x, s[4 * i], fmaf(k.x, v, -au.x * dot));
      s[4 * i + 1] = fmaf(w.y, s[4 * i + 1], fmaf(k.y, v, -au.y * dot));
      s[4 * i + 2] = fmaf(w.z, s[4 * i + 2], fmaf(k.z, v, -au.z * dot));
      s[4 * i + 3] = fmaf(w.w, s[4 * i + 3], fmaf(k.w, v, -au.w * dot));
      o0 = fmaf(r.x, s[4 * i], o0);
      o1 = fmaf(r.y, s[4 * i + 1], o1);
      o2 = fmaf(r.z, s[4 * i + 2], o2);
      o3 = fmaf(r.w, s[4 * i + 3], o3);
    }
    if (live) out[(size_t)t * out_stride + base + column] = (o0 + o1) + (o2 + o3);
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (request_active[request] && live) {
#pragma unroll
    for (int i = 0; i < P; ++i)
      if (i < dim) s_base[(size_t)i * dim + column] = s[i];
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
extern "C" int cie_delta_stream_max_dim() { return cie::kDeltaStreamMaxDim; }

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
  const int columns = dim < kDeltaBlockColumns ? dim : kDeltaBlockColumns;
  const int threads = (kDeltaLanes * columns + 31) / 32 * 32;
  const dim3 grid(requests, heads, (dim + kDeltaBlockColumns - 1) / kDeltaBlockColumns);
#define CIE_DELTA_SCAN(R)                                                                                        \
  CIE_LAUNCH("delta_scan", delta_scan_kernel<R>, grid, dim3(threads), 0, (cudaStream_t)stream, proj, proj_stride, \
             r_off, k_off, v_off, a_off, decay, decay_stride, decay_bias, removal_bias, out, out_stride, state,  \
             query_start, slots, request_active, heads, dim, max_slots, err)
  if (dim <= 32) { CIE_DELTA_SCAN(4); }
  else if (dim <= 64) { CIE_DELTA_SCAN(8); }
  else if (dim <= 128) { CIE_DELTA_SCAN(16); }
  else { CIE_DELTA_SCAN(32); }
#undef CIE_DELTA_SCAN
  return 0;
}

// Floats of scratch memory the two-kernel form wants for `tokens` tokens.
extern "C" long long cie_delta_stream_floats(int tokens, int heads, int dim) {
  const int pad = dim <= 32 ? 32 : dim <= 64 ? 64 : 128;
  return (long long)tokens * heads * cie::kDeltaFields * pad;
}

extern "C" int cie_delta_stream(const float* proj, int proj_stride, int r_off, int k_off, int v_off, int a_off,
                                const float* decay, int decay_stride, const float* decay_bias,
                                const float* removal_bias, float* packed, float* out, int out_stride, float* state,
                                const int* query_start, const int* slots, const int* request_active, int tokens,
                                int requests, int heads, int dim, int max_slots, int* err, void* stream) {
  using namespace cie;
  if (requests <= 0 || tokens <= 0) return 0;
  if (dim < 1 || dim > kDeltaStreamMaxDim) CIE_FAIL("delta_stream: head size %d is outside 1..%d", dim, kDeltaStreamMaxDim);
  const int pad = dim <= 32 ? 32 : dim <= 64 ? 64 : 128;
  CIE_LAUNCH("delta_prepare", delta_prepare_kernel, dim3(tokens, heads), dim3(32), 0, (cudaStream_t)stream, proj,
             proj_stride, r_off, k_off, v_off, a_off, decay, decay_stride, decay_bias, removal_bias, packed, tokens, heads,
             dim, pad);
  const int threads = (dim + 31) / 32 * 32;
  const dim3 grid(requests, heads);
#define CIE_DELTA_STREAM(P)                                                                                       \
  CIE_LAUNCH("delta_stream", delta_stream_kernel<P>, grid, dim3(threads), 0, (cudaStream_t)stream, packed, out,   \
             out_stride, state, query_start, slots, request_active, tokens, heads, dim, max_slots, err)
  if (pad == 32) { CIE_DELTA_STREAM(32); }
  else if (pad == 64) { CIE_DELTA_STREAM(64); }
  else { CIE_DELTA_STREAM(128); }
#undef CIE_DELTA_STREAM
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
