// The grouped products of routed experts on the 5th-generation tensor cores.
//
// The (token, expert) pairs of a step are grouped by expert on the device (moe.cu: places, tiles of
// up to 128 rows of one expert).  Here a CTA takes one such tile and 128 output columns: the tile's
// rows and the expert's weight rows come by TMA (128-byte swizzle) into a three-stage ring, one
// thread issues tcgen05.mma into a float32 accumulator in tensor memory, and the four warps read
// it back with tcgen05.ld for the epilogue.  Rows must lie one after another for TMA, so the
// gate/up product first gathers the tokens' rows by place (one memory-bound kernel); the down
// product reads the activations, which the gate/up product wrote by place.
//
//   gate_up  W = [experts][2F][H], gate and up rows of an expert interleaved in blocks of 16 (16 gate
//            rows, their 16 up rows, ...): a thread holds both halves of SiLU(gate) * up and writes
//            act[place][channel] (bfloat16)
//   down     W = [experts][H][F]; the result goes, float32, to the row of the tile row's pair
//
// A tile's rows beyond the expert's last (they belong to the next expert, or lie outside the buffer
// and read as zero) and columns beyond the expert's last are computed and never stored.  Two CTAs
// share an SM (97 KB of shared memory and 128 tensor-memory columns each), so one CTA's epilogue
// runs beside the other's products.  Every wait on an mbarrier is bounded.
#include "blackwell.cuh"
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

using namespace bw;
using bf16 = __nv_bfloat16;

constexpr int BM = 128, BK = 64, UMMA_K = 16, STAGES = 3;
constexpr int A_STAGE_BYTES = BM * BK * 2;
// BN, the output columns of a tile, is 128 (two CTAs an SM) or, on request, 256 (one CTA an SM; a third
// less operand traffic per product, but nothing beside a tile's set-up and epilogue)
template <int BN> constexpr int stage_bytes() { return A_STAGE_BYTES + BN * BK * 2; }
template <int BN> constexpr size_t smem_bytes() { return (size_t)STAGES * stage_bytes<BN>() + 1024; }

__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// sorted[p] = x[place_to_pair[p] / top], 16 bytes a thread.
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, bf16* __restrict__ sorted,
                                       const int* __restrict__ place_to_pair, int pairs, int top, int hidden) {
  pdl_wait();
  pdl_trigger();
  const int pieces = hidden / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)pairs * pieces;
       i += (long long)gridDim.x * blockDim.x) {
    const int p = (int)(i / pieces), c = (int)(i % pieces);
    const int token = place_to_pair[p] / top;
    reinterpret_cast<uint4*>(sorted + (size_t)p * hidden)[c] = reinterpret_cast<const uint4*>(x + (size_t)token * hidden)[c];
  }
}

struct GroupedArgs {
  void* out;
  const int* place_to_pair;
  const int* tiles;        // (expert, first place, rows) per tile
  const int* tile_count;
  int rows_per_expert;     // weight rows of one expert (2F or H)
  int n;                   // output columns of a row (F or H)
  int k;
  int* err;
};

template <bool kGateUp, int BN>
__global__ void __launch_bounds__(128) moe_grouped_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                   const __grid_constant__ CUtensorMap map_b,
                                                                   const GroupedArgs a) {
  constexpr int STAGE_BYTES = stage_bytes<BN>();
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* stage_base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_bar;
  __shared__ uint32_t tmem_base_s;

  pdl_wait();
  pdl_trigger();
  if ((int)blockIdx.y >= a.tile_count[0]) return;       // the grid holds the most tiles a step can have
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int expert = a.tiles[3 * blockIdx.y], place0 = a.tiles[3 * blockIdx.y + 1], rows = a.tiles[3 * blockIdx.y + 2];
  const int col0_tile = blockIdx.x * BN;                 // first weight row of the tile inside the expert
  const int b_row0 = expert * a.rows_per_expert + col0_tile;
  const int k_tiles = (a.k + BK - 1) / BK;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_init_fence();
  }
  if (warp == 0) {
    __syncwarp();
    tmem_alloc<BN>(&tmem_base_s);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    if (lane == 0) {     // copies
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        const uint32_t phase = (kt / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], phase ^ 1, a.err)) break;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        unsigned char* dst = stage_base + (size_t)s * STAGE_BYTES;
        tma_load_2d(dst, &map_a, &full_bar[s], kt * BK, place0);
        tma_load_2d(dst + A_STAGE_BYTES, &map_b, &full_bar[s], kt * BK, b_row0);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {     // products
      constexpr uint32_t idesc = idesc_bf16(BM, BN);
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % STAGES;
        const uint32_t phase = (kt / STAGES) & 1;
        if (!mbar_wait(&full_bar[s], phase, a.err)) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(stage_base + (size_t)s * STAGE_BYTES);
        const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_STAGE_BYTES);
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma_bf16(tmem_base, a_desc + 2 * kk, b_desc + 2 * kk, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
        tc_commit(&empty_bar[s]);
      }
      tc_commit(&acc_bar);
    }
    __syncwarp();
  }

  // ---- epilogue: warp w reads tensor-memory lanes 32w .. 32w + 31 (rows of the tile)
  const bool ready = mbar_wait(&acc_bar, 0, a.err);
  tc_fence_after();
  const int r = warp * 32 + lane;
  if (ready) {
    const bool live = r < rows;
    const uint32_t lane_base = tmem_base + ((uint32_t)(warp * 32) << 16);
    if constexpr (kGateUp) {
      bf16* dst_row = reinterpret_cast<bf16*>(a.out) + (size_t)(place0 + r) * a.n;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t gate[16], up[16];
        tmem_load16(lane_base + c0, gate);          // every lane of the warp takes part in the load
        tmem_load16(lane_base + c0 + 16, up);
        const int channel0 = (col0_tile + c0) / 2;  // 32 interleaved rows hold 16 channels
        if (!live || channel0 >= a.n) continue;
        if (channel0 + 16 <= a.n) {
          uint32_t packed[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g0 = __uint_as_float(gate[2 * j]), g1 = __uint_as_float(gate[2 * j + 1]);
            const float v0 = g0 / (1.f + expf(-g0)) * __uint_as_float(up[2 * j]);
            const float v1 = g1 / (1.f + expf(-g1)) * __uint_as_float(up[2 * j + 1]);
            __nv_bfloat162 pair = __floats2bfloat162_rn(v0, v1);
            packed[j] = *reinterpret_cast<uint32_t*>(&pair);
          }
          reinterpret_cast<uint4*>(dst_row + channel0)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          reinterpret_cast<uint4*>(dst_row + channel0)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
          for (int j = 0; j < 16 && channel0 + j < a.n; ++j) {
            const float g = __uint_as_float(gate[j]);
            dst_row[channel0 + j] = __float2bfloat16_rn(g / (1.f + expf(-g)) * __uint_as_float(up[j]));
          }
        }
      }
    } else {
      const int pair = live ? a.place_to_pair[place0 + r] : 0;
      float* dst_row = reinterpret_cast<float*>(a.out) + (size_t)pair * a.n;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t raw[16];
        tmem_load16(lane_base + c0, raw);
        const int col0 = col0_tile + c0;
        if (!live || col0 >= a.n) continue;
        if (col0 + 16 <= a.n) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<float4*>(dst_row + col0)[j] =
                make_float4(__uint_as_float(raw[4 * j]), __uint_as_float(raw[4 * j + 1]),
                            __uint_as_float(raw[4 * j + 2]), __uint_as_float(raw[4 * j + 3]));
        } else {
          for (int j = 0; j < 16 && col0 + j < a.n; ++j) dst_row[col0 + j] = __uint_as_float(raw[j]);
        }
      }
    }
  } else {
    // a wait ran out: give copies that may still be in flight time to land before leaving
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_free<BN>(tmem_base);
}

template <bool kGateUp, int BN>
static int launch_grouped(const CUtensorMap& map_a, const CUtensorMap& map_b, const GroupedArgs& a, dim3 grid,
                          cudaStream_t stream) {
  constexpr size_t smem = smem_bytes<BN>();
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(moe_grouped_tcgen05_kernel<kGateUp, BN>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (status != cudaSuccess) CIE_FAIL("moe_tcgen05: shared memory %zu: %s", smem, cudaGetErrorString(status));
    configured = true;
  }
  CIE_LAUNCH("moe_tcgen05", (moe_grouped_tcgen05_kernel<kGateUp, BN>), grid, dim3(128), smem, stream, map_a, map_b, a);
  return 0;
}

// 128 columns a tile; CIE_MOE_TILE_COLUMNS=256 asks for the wider tile (measured slower: with one CTA an SM
// nothing runs beside a tile's set-up and epilogue, 5.63 against 5.41 ms for a 2,048-token prefill)
static int tile_columns(int) {
  static const int forced = [] { const char* v = getenv("CIE_MOE_TILE_COLUMNS"); return v ? atoi(v) : 0; }();
  return forced == 256 ? 256 : 128;
}

}  // namespace cie

using namespace cie;

// x: [tokens][hidden]; sorted: scratch [tokens * top][hidden]; w_gate_up: [experts][2 ff][hidden], gate
// and up rows interleaved in blocks of 16; act: [tokens * top][ff], rows by place.  All bfloat16,
// 16-byte aligned; hidden a multiple of 8, ff a multiple of 16.
extern "C" int cie_moe_gate_up_tcgen05(const void* x, void* sorted, const void* w_gate_up, void* act,
                                       const int* place_to_pair, const int* tiles, const int* tile_count,
                                       int tokens, int top, int experts, int ff, int hidden, int row_tile,
                                       int* err, void* stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8 || ff % 16) CIE_FAIL("moe_gate_up_tcgen05: sizes %d / %d", hidden, ff);
  if (row_tile != BM) CIE_FAIL("moe_gate_up_tcgen05: tiles of %d rows, this kernel takes %d", row_tile, BM);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(sorted) | reinterpret_cast<uintptr_t>(w_gate_up) |
       reinterpret_cast<uintptr_t>(act)) & 15)
    CIE_FAIL("moe_gate_up_tcgen05: operands must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  const int pairs = tokens * top;
  const long long pieces = (long long)pairs * (hidden / 8);
  int blocks = (int)((pieces + 255) / 256);
  if (blocks > 148 * 8) blocks = 148 * 8;
  CIE_LAUNCH("moe_gather_rows", moe_gather_rows_kernel, dim3(blocks), dim3(256), 0, s, (const bf16*)x, (bf16*)sorted,
             place_to_pair, pairs, top, hidden);
  const int bn = tile_columns(pairs);
  CUtensorMap map_a, map_b;
  if (!tensor_map_bf16(sorted, pairs, hidden, BM, &map_a) ||
      !tensor_map_bf16(w_gate_up, (long long)experts * 2 * ff, hidden, bn, &map_b))
    CIE_FAIL("moe_gate_up_tcgen05: cuTensorMapEncodeTiled failed");
  GroupedArgs a = {act, place_to_pair, tiles, tile_count, 2 * ff, ff, hidden, err};
  const int max_tiles = (pairs + BM - 1) / BM + experts;
  const dim3 grid((2 * ff + bn - 1) / bn, max_tiles);
  return bn == 256 ? launch_grouped<true, 256>(map_a, map_b, a, grid, s) : launch_grouped<true, 128>(map_a, map_b, a, grid, s);
}

// act: [tokens * top][ff] by place; w_down: [experts][hidden][ff]; rows: float32 [tokens * top][hidden],
// the row of pair (t, j) at t * top + j.
extern "C" int cie_moe_down_tcgen05(const void* act, const void* w_down, float* rows, const int* place_to_pair,
                                    const int* tiles, const int* tile_count, int tokens, int top, int experts,
                                    int ff, int hidden, int row_tile, int* err, void* stream) {
  if (tokens <= 0) return 0;
  if (hidden % 8 || ff % 8) CIE_FAIL("moe_down_tcgen05: sizes %d / %d", hidden, ff);
  if (row_tile != BM) CIE_FAIL("moe_down_tcgen05: tiles of %d rows, this kernel takes %d", row_tile, BM);
  if ((reinterpret_cast<uintptr_t>(act) | reinterpret_cast<uintptr_t>(w_down) | reinterpret_cast<uintptr_t>(rows)) & 15)
    CIE_FAIL("moe_down_tcgen05: operands must be 16-byte aligned");
  const int pairs = tokens * top;
  const int bn = tile_columns(pairs);
  CUtensorMap map_a, map_b;
  if (!tensor_map_bf16(act, pairs, ff, BM, &map_a) ||
      !tensor_map_bf16(w_down, (long long)experts * hidden, ff, bn, &map_b))
    CIE_FAIL("moe_down_tcgen05: cuTensorMapEncodeTiled failed");
  GroupedArgs a = {rows, place_to_pair, tiles, tile_count, hidden, hidden, ff, err};
  const int max_tiles = (pairs + BM - 1) / BM + experts;
  const dim3 grid((hidden + bn - 1) / bn, max_tiles);
  cudaStream_t s = (cudaStream_t)stream;
  return bn == 256 ? launch_grouped<false, 256>(map_a, map_b, a, grid, s) : launch_grouped<false, 128>(map_a, map_b, a, grid, s);
}
