// Triangle-multiplication contraction for sm_100a: per batch item b and hidden channel d
//   x[b, d, i, j] = sum_k a[b, d, i, k] * b[b, d, j, k]
// i.e. 128 * B independent [N x N] = [N x N] · [N x N]ᵀ bf16 GEMMs with fp32 accumulation.  The projection kernel
// writes a and b channel-major with the contraction index k contiguous (for the incoming node it walks the pair
// tensor through swapped strides, so the same layout serves both directions), so both operands are K-major.
//
// One CTA computes [128 x 256] output tiles: TMA loads [128 x 64] / [256 x 64] operand tiles into a four-stage
// ring, one thread issues tcgen05.mma (M 128, N 256, K 16) into one of two TMEM accumulators, and four epilogue
// warps (TMEM lane = output row) convert the finished accumulator to bf16 and write 512 contiguous bytes per
// thread while the next tile's MMAs run.
//
// Warp roles (192 threads): warps 0-3 epilogue, warp 4 TMA producer, warp 5 MMA issuer / TMEM owner.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kThreads = 192;
constexpr int kBM = 128, kBN = 256, kBK = 64;
constexpr int kStages = 4;
constexpr int kStageBytes = (kBM + kBN) * kBK * 2;  // 48 KiB
constexpr int kSmBars = kStages * kStageBytes;
enum Bar { FULL = 0, EMPTY = kStages, ACC_FULL = 2 * kStages, ACC_EMPTY = 2 * kStages + 2, NUM_BARS = 2 * kStages + 4 };
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

struct ContractParams {
  int N;          // tokens
  int planes;     // B * hidden
  int hidden;     // channels per batch item (a planes first, b planes next)
  int tiles_m, tiles_n, num_tiles;
  __nv_bfloat16* x;
  long long x_plane, x_row;  // element strides of x[plane][i][j]
  int* status;
};

struct Tile {
  int plane, a_plane, b_plane, m0, n0;
};
__device__ __forceinline__ Tile decode_tile(const ContractParams& p, int t) {
  Tile r;
  const int nt = t % p.tiles_n;
  t /= p.tiles_n;
  const int mt = t % p.tiles_m;
  r.plane = t / p.tiles_m;
  const int b = r.plane / p.hidden, d = r.plane - b * p.hidden;
  r.a_plane = b * 2 * p.hidden + d;
  r.b_plane = r.a_plane + p.hidden;
  r.m0 = mt * kBM, r.n0 = nt * kBN;
  return r;
}

// 32-byte store; the address must be 32-byte aligned.
__device__ __forceinline__ void stg256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
trimul_contract_kernel(const __grid_constant__ CUtensorMap tm_ab, const ContractParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kSmBars;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + kSmBars + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + kSmBars + NUM_BARS * 8 + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag[0] = 0, abort_flag[1] = 0;
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bars + (FULL + i) * 8, 1);
      mbar_init(bars + (EMPTY + i) * 8, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + (ACC_FULL + i) * 8, 1);
      mbar_init(bars + (ACC_EMPTY + i) * 8, 4);
    }
    fence_mbar_init();
  }
  if (warp == 5) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int my_tiles = (p.num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;
  const int ksteps = (p.N + kBK - 1) / kBK;

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_ab);
      int g = 0;  // ring position
      bool ok = true;
      for (int i = 0; ok && i < my_tiles; ++i) {
        const Tile t = decode_tile(p, blockIdx.x + i * gridDim.x);
        for (int ks = 0; ks < ksteps; ++ks, ++g) {
          const int stage = g % kStages;
          ok = mbar_wait(bars + (EMPTY + stage) * 8, ((g / kStages) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t full = bars + (FULL + stage) * 8;
          const uint32_t sa = base + stage * kStageBytes;
          mbar_expect_tx(full, kStageBytes);
          tma_load_3d(sa, &tm_ab, full, ks * kBK, t.m0, t.a_plane);
          tma_load_3d(sa + kBM * kBK * 2, &tm_ab, full, ks * kBK, t.n0, t.b_plane);
          tma_load_3d(sa + kBM * kBK * 2 + 128 * kBK * 2, &tm_ab, full, ks * kBK, t.n0 + 128, t.b_plane);
        }
      }
      // If the loop was abandoned, give copies still in flight a bounded chance to land.
      if (*abort_flag && g > 0) mbar_wait(bars + (FULL + (g - 1) % kStages) * 8, ((g - 1) / kStages) & 1, abort_flag + 1);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, kBN);
      int g = 0;
      bool ok = true;
      for (int i = 0; ok && i < my_tiles; ++i) {
        const int slot = i & 1;
        ok = mbar_wait(bars + (ACC_EMPTY + slot) * 8, ((i >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem_base + slot * kBN;
        for (int ks = 0; ks < ksteps; ++ks, ++g) {
          const int stage = g % kStages;
          ok = mbar_wait(bars + (FULL + stage) * 8, (g / kStages) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint32_t sa = base + stage * kStageBytes;
          // [rows][64 k] tiles with 128-byte swizzle: 8-row groups 1 KiB apart; a K step of 16 = 32 bytes
          const uint64_t da = make_smem_desc(sa, 16, 1024, kLayoutSw128);
          const uint64_t db = make_smem_desc(sa + kBM * kBK * 2, 16, 1024, kLayoutSw128);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) umma_ss(d, da + k * 2, db + k * 2, idesc, (ks > 0 || k > 0) ? 1u : 0u);
          umma_commit(bars + (EMPTY + stage) * 8);  // the stage is free once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(bars + (ACC_FULL + slot) * 8);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int m = warp * 32 + lane;  // output row inside the tile == TMEM lane
    const uint32_t lane_taddr = tmem_base + (uint32_t(warp * 32) << 16);
    bool ok = true;
    for (int i = 0; ok && i < my_tiles; ++i) {
      const Tile t = decode_tile(p, blockIdx.x + i * gridDim.x);
      const int slot = i & 1;
      ok = mbar_wait(bars + (ACC_FULL + slot) * 8, (i >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const int row = t.m0 + m;
      __nv_bfloat16* dst = p.x + t.plane * p.x_plane + (long long)row * p.x_row + t.n0;
      uint32_t acc[2][32];
      tmem_ld32(lane_taddr + slot * kBN, acc[0]);
#pragma unroll
      for (int g = 0; g < kBN / 32; ++g) {
        tmem_ld_wait();
        if (g + 1 < kBN / 32) tmem_ld32(lane_taddr + slot * kBN + (g + 1) * 32, acc[(g + 1) & 1]);
        const uint32_t (&a)[32] = acc[g & 1];
        uint32_t packed[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) packed[j] = pack_bf16x2(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1]));
        // columns past the row pitch are never written; columns between N and the pitch receive zeros (the
        // operand rows past N are zero-filled by the TMA loads)
        if (row < p.N) {
          if (t.n0 + g * 32 + 16 <= p.x_row) stg256(dst + g * 32, packed);
          if (t.n0 + g * 32 + 32 <= p.x_row) stg256(dst + g * 32 + 16, packed + 8);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (ACC_EMPTY + slot) * 8);
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_trimul_contract(const void* ab, void* x, int B, int N, int64_t pitch, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(ab && x, "trimul_contract: NULL pointer");
  B200TA_REQUIRE(B > 0 && N > 0, "trimul_contract: bad sizes B=%d N=%d", B, N);
  B200TA_REQUIRE(pitch >= N && pitch % 16 == 0, "trimul_contract: pitch=%lld must be a multiple of 16 and >= N=%d",
                 (long long)pitch, N);
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(ab) & 31u) == 0 && (reinterpret_cast<uintptr_t>(x) & 31u) == 0,
                 "trimul_contract: buffers must be 32-byte aligned");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  constexpr int kHidden = kC;
  CUtensorMap tm_ab;
  {
    // (k, row, plane): rows and k past N read as zero
    uint64_t dims[3] = {uint64_t(N), uint64_t(N), uint64_t(B) * 2 * kHidden};
    uint64_t strides[2] = {uint64_t(pitch) * 2, uint64_t(pitch) * N * 2};
    uint32_t box[3] = {kBK, 128, 1};
    rc = encode_tensor_map(&tm_ab, ab, 2, 3, dims, strides, box, SWZ_128, "trimul a/b planes");
    if (rc != B200TA_OK) return rc;
  }
  ContractParams p{};
  p.N = N, p.planes = B * kHidden, p.hidden = kHidden;
  p.tiles_m = (N + kBM - 1) / kBM, p.tiles_n = (N + kBN - 1) / kBN;
  const int64_t tiles = int64_t(p.planes) * p.tiles_m * p.tiles_n;
  B200TA_REQUIRE(tiles < (int64_t(1) << 31), "trimul_contract: too many tiles");
  p.num_tiles = int(tiles);
  p.x = static_cast<__nv_bfloat16*>(x);
  p.x_row = pitch, p.x_plane = pitch * N;
  p.status = st->status_dev;

  B200TA_CHECK_CUDA(cudaFuncSetAttribute(trimul_contract_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  trimul_contract_kernel<<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_ab, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
