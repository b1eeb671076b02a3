// Pair bias of the single-track attention (sm_100a): bias[b,h,q,k] = scale * LayerNorm(z[b,q,k,:]) · W_z[h,:].
//
// One pass over the pair tensor, bound by reading it (256 bytes per position in, 2 bytes per head out).  A
// persistent CTA per SM walks 128-position tiles; each tile arrives by TMA into a ring of six 32 KiB stages (deep
// enough to keep the SM's share of the HBM bandwidth in flight), four warps compute the LayerNorm statistics of
// their rows from the shared-memory copy while one tcgen05.mma (N = 16) multiplies the raw rows with the
// LayerNorm-folded head weights, and the same four warps finish
//     bias = rstd * acc - mean * rstd * rowsum[h] + const[h]
// and store it head-major with the key axis innermost (zeros in the key padding).  Two such warpgroups take
// alternate tiles (each owns one of the two TMEM accumulators), so every scheduler has two warps to switch between.
//
// Warp roles (320 threads): warps 0-7 statistics + output (TMEM lane = position), warp 8 TMA producer,
// warp 9 MMA issuer / TMEM owner.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kTileM = 128;
constexpr int kStages = 6;
constexpr int kThreads = 320;
constexpr int kMaxHeads = 16;
constexpr int kFirstRow = 4 * kHeads * kHeadDim;  // the bias heads follow the q, k, v, g rows of a node pack

struct PairBiasParams {
  int B, Q, K, K_pad;
  int tiles_k;
  int num_tiles;
  int heads;
  const float2* sc;  // {rowsum, const} of the folded head rows
  const int* flags;  // flags[0] != 0 -> apply LayerNorm statistics
  float eps;
  __nv_bfloat16* bias;
  long long bs_b, bs_h, bs_q, bs_k;
  int* status;
};

constexpr int kSmA = 0;                               // kStages x 32 KiB
constexpr int kSmW = kSmA + kStages * 32768;          // 2 channel halves x [16 heads][64 ch]
constexpr int kSmSc = kSmW + 2 * kMaxHeads * 128;     // 8 x {rowsum0, rowsum1, const0, const1}
constexpr int kSmBars = kSmSc + (kMaxHeads / 2) * 16;
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

enum Bar { W_FULL = 0, A_FULL = 1, A_EMPTY = A_FULL + kStages, ACC_FULL = A_EMPTY + kStages, ACC_EMPTY = ACC_FULL + 2,
           NUM_BARS = ACC_EMPTY + 2 };

__global__ void __launch_bounds__(kThreads, 1)
pair_bias_kernel(const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_w, const PairBiasParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kSmBars;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + kSmBars + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + kSmBars + NUM_BARS * 8 + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    mbar_init(bars + W_FULL * 8, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bars + (A_FULL + i) * 8, 1);
      mbar_init(bars + (A_EMPTY + i) * 8, 5);  // 4 statistics warps + the MMA commit
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + (ACC_FULL + i) * 8, 1);
      mbar_init(bars + (ACC_EMPTY + i) * 8, 4);
    }
    fence_mbar_init();
  }
  if (threadIdx.x < kMaxHeads / 2) {
    const float2 a = p.sc[kFirstRow + 2 * threadIdx.x], b = p.sc[kFirstRow + 2 * threadIdx.x + 1];
    reinterpret_cast<float4*>(gen + kSmSc)[threadIdx.x] = make_float4(a.x, b.x, a.y, b.y);
  }
  if (warp == 9) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 32);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int my_tiles = (p.num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;  // blockIdx.x < num_tiles

  if (warp == 8) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_z);
      tma_prefetch_desc(&tm_w);
      mbar_expect_tx(bars + W_FULL * 8, 2 * kMaxHeads * 128);
      for (int kh = 0; kh < 2; ++kh)
        tma_load_2d(base + kSmW + kh * kMaxHeads * 128, &tm_w, bars + W_FULL * 8, kh * 64, kFirstRow);
      int issued = 0;
      for (int i = 0; i < my_tiles; ++i) {
        const int tile = blockIdx.x + i * gridDim.x;
        const int kt = tile % p.tiles_k;
        const int bq = tile / p.tiles_k;
        const int stage = i % kStages;
        if (!mbar_wait(bars + (A_EMPTY + stage) * 8, ((i / kStages) & 1) ^ 1, abort_flag)) break;
        const uint32_t full = bars + (A_FULL + stage) * 8;
        mbar_expect_tx(full, 32768);
        tma_load_4d(base + kSmA + stage * 32768, &tm_z, full, 0, kt * kTileM, bq % p.Q, bq / p.Q);
        tma_load_4d(base + kSmA + stage * 32768 + 16384, &tm_z, full, 64, kt * kTileM, bq % p.Q, bq / p.Q);
        ++issued;
      }
      // If the loop was abandoned, give copies still in flight a bounded chance to land.
      if (*abort_flag)
        for (int j = issued > kStages ? issued - kStages : 0; j < issued; ++j)
          mbar_wait(bars + (A_FULL + j % kStages) * 8, (j / kStages) & 1, abort_flag + 1);
    }
  } else if (warp == 9) {
    if (lane == 0) {
      bool ok = mbar_wait(bars + W_FULL * 8, 0, abort_flag);
      const uint32_t idesc = make_idesc_bf16(kTileM, kMaxHeads);
      for (int i = 0; ok && i < my_tiles; ++i) {
        const int stage = i % kStages, slot = i & 1;
        ok = mbar_wait(bars + (A_FULL + stage) * 8, (i / kStages) & 1, abort_flag) &&
             mbar_wait(bars + (ACC_EMPTY + slot) * 8, ((i >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = make_smem_desc(base + kSmA + stage * 32768, 16, 1024, kLayoutSw128);
        const uint64_t db = make_smem_desc(base + kSmW, 16, 1024, kLayoutSw128);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(tmem_base + slot * kMaxHeads, da + ((k >> 2) * (16384 >> 4) + (k & 3) * 2),
                  db + ((k >> 2) * ((kMaxHeads * 128) >> 4) + (k & 3) * 2), idesc, k > 0 ? 1u : 0u);
        umma_commit(bars + (ACC_FULL + slot) * 8);
        umma_commit(bars + (A_EMPTY + stage) * 8);
      }
    }
  } else {
    const int wg = warp >> 2;               // this warpgroup takes the tiles i with i % 2 == wg
    const int m = (warp & 3) * 32 + lane;  // row of the tile == TMEM lane
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const bool normalize = __ldg(p.flags) != 0;
    const float4* sc4 = reinterpret_cast<const float4*>(gen + kSmSc);
    bool ok = true;
    for (int i = wg; ok && i < my_tiles; i += 2) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int kt = tile % p.tiles_k;
      const int bq = tile / p.tiles_k;
      const int q = bq % p.Q, b = bq / p.Q;
      const int stage = i % kStages, slot = wg;
      const int k = kt * kTileM + m;  // this thread's key position
      ok = mbar_wait(bars + (A_FULL + stage) * 8, (i / kStages) & 1, abort_flag);
      if (!ok) break;
      float rstd = 1.f, nmr = 0.f;
      if (normalize) {
        // LayerNorm statistics of row m from the swizzled smem copy of the z tile.
        uint32_t v[64];
        const uint32_t a0 = base + kSmA + stage * 32768;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          uint4 x = lds128(a0 + (c >> 3) * 16384 + sw128_offset(m, c & 7));
          v[c * 4 + 0] = x.x, v[c * 4 + 1] = x.y, v[c * 4 + 2] = x.z, v[c * 4 + 3] = x.w;
        }
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 64; ++j) sum4[j & 3] += bf16_lo(v[j]) + bf16_hi(v[j]);
        const float mu = ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3])) * (1.f / kC);
        float var4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          const float d0 = bf16_lo(v[j]) - mu, d1 = bf16_hi(v[j]) - mu;
          var4[j & 3] = fmaf(d0, d0, var4[j & 3]);
          var4[j & 3] = fmaf(d1, d1, var4[j & 3]);
        }
        rstd = rsqrtf(((var4[0] + var4[1]) + (var4[2] + var4[3])) * (1.f / kC) + p.eps);
        nmr = -mu * rstd;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (A_EMPTY + stage) * 8);  // done reading the z tile
      ok = mbar_wait(bars + (ACC_FULL + slot) * 8, (i >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t a[16];
      tmem_ld16(lane_taddr + slot * kMaxHeads, a);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (ACC_EMPTY + slot) * 8);
      if (k < p.K_pad) {
        __nv_bfloat16* dst = p.bias + b * p.bs_b + q * p.bs_q + k * p.bs_k;
#pragma unroll
        for (int hp = 0; hp < kMaxHeads / 2; ++hp) {
          if (2 * hp >= p.heads) break;
          const float4 t = sc4[hp];  // {rowsum0, rowsum1, const0, const1}
          const float v0 = k < p.K ? fmaf(rstd, __uint_as_float(a[2 * hp]), fmaf(nmr, t.x, t.z)) : 0.f;
          const float v1 = k < p.K ? fmaf(rstd, __uint_as_float(a[2 * hp + 1]), fmaf(nmr, t.y, t.w)) : 0.f;
          dst[(2 * hp) * p.bs_h] = __float2bfloat16_rn(v0);
          dst[(2 * hp + 1) * p.bs_h] = __float2bfloat16_rn(v1);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 32);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_pair_bias(const void* z, int64_t zs_b, int64_t zs_q, int64_t zs_k, const void* packed, float eps,
                     void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q, int64_t bs_k, int num_heads, int B, int Q,
                     int K, int K_pad, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(z && packed && bias, "pair_bias: NULL pointer");
  B200TA_REQUIRE(num_heads > 0 && num_heads <= kMaxHeads && num_heads % 2 == 0,
                 "pair_bias: num_heads=%d must be even and at most %d", num_heads, kMaxHeads);
  B200TA_REQUIRE(B > 0 && Q > 0 && K > 0 && K_pad >= K, "pair_bias: bad sizes B=%d Q=%d K=%d K_pad=%d", B, Q, K, K_pad);
  B200TA_REQUIRE(int64_t(B) * Q < (int64_t(1) << 31), "pair_bias: B*Q too large");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "pair_bias: packed must be 256-byte aligned");
  B200TA_REQUIRE(zs_b % 8 == 0 && zs_q % 8 == 0 && zs_k % 8 == 0 && zs_b >= 0 && zs_q >= 0 && zs_k >= 0,
                 "pair_bias z: element strides must be non-negative multiples of 8 (16 bytes)");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;
  const char* pk = static_cast<const char*>(packed);

  CUtensorMap tm_z, tm_w;
  {
    // dims (c, k, q, b); a size-1 dimension may carry any stride: give it a valid one
    auto fix = [](int64_t stride, int extent) -> uint64_t { return extent == 1 ? 256u : uint64_t(stride) * 2u; };
    uint64_t dims[4] = {uint64_t(kC), uint64_t(K), uint64_t(Q), uint64_t(B)};
    uint64_t strides[3] = {fix(zs_k, K), fix(zs_q, Q), fix(zs_b, B)};
    uint32_t box[4] = {64, kTileM, 1, 1};
    rc = encode_tensor_map(&tm_z, z, 2, 4, dims, strides, box, SWZ_128, "pair_bias z");
    if (rc != B200TA_OK) return rc;
  }
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(kNodeRows)};
    uint64_t strides[1] = {uint64_t(kC) * 2};
    uint32_t box[2] = {64, kMaxHeads};
    rc = encode_tensor_map(&tm_w, pk + kNodeWOff, 2, 2, dims, strides, box, SWZ_128, "pair_bias weights");
    if (rc != B200TA_OK) return rc;
  }
  PairBiasParams p{};
  p.B = B, p.Q = Q, p.K = K, p.K_pad = K_pad;
  p.tiles_k = (K + kTileM - 1) / kTileM;
  p.num_tiles = B * Q * p.tiles_k;
  p.heads = num_heads;
  p.sc = reinterpret_cast<const float2*>(pk + kNodeScOff);
  p.flags = reinterpret_cast<const int*>(pk + kNodeFlagsOff);
  p.eps = eps;
  p.bias = static_cast<__nv_bfloat16*>(bias);
  p.bs_b = bs_b, p.bs_h = bs_h, p.bs_q = bs_q, p.bs_k = bs_k;
  p.status = st->status_dev;
  B200TA_CHECK_CUDA(cudaFuncSetAttribute(pair_bias_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  pair_bias_kernel<<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_z, tm_w, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
