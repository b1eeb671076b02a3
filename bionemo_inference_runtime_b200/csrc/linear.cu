// Dense layers of the single track (sm_100a): out = finish(A · Wᵀ) for a few thousand rows.
//
// The single representation has one row per token, so its projections are small GEMMs (M = tokens, K and N a few
// hundred to a few thousand).  One CTA computes one 128x128 output tile: a TMA warp streams 64-wide K steps of A
// and W through a 4-stage ring, one thread issues tcgen05.mma into a TMEM accumulator, and four warps finish the
// rows (one TMEM lane = one row = one thread):
//
//   value[n] = rstd * acc[n] + nmr * rowsum[n] + const[n]        (LayerNorm folded into W; rstd = 1, nmr = 0 without)
//
//   kPlanes: columns are (which, head, 32) with 16 heads: written head-major as [which][B][16][rows][32]; the last
//            plane as sigmoid(value) (the gate factors the attention kernel multiplies with).
//   kRows:   out[b, row, n] = value[n] (+ residual[b, row, n]).
//   kSwiglu: every 32 columns hold 16 values and their 16 gates: out[b, row, n/2 ..] = silu(gate) * value.
//
// Warp roles (192 threads): warps 0-3 finish rows, warp 4 TMA producer, warp 5 MMA issuer / TMEM owner.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kTile = 128;
constexpr int kStepK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kStageBytes = 2 * kTile * kStepK * 2;  // A and W blocks of one K step

enum Mode { kPlanes = 0, kRows = 1, kSwiglu = 2 };

struct LinearParams {
  int B, rows, K, N;
  int tiles_m;       // row tiles per batch item
  const float2* sc;  // [N] {rowsum, const}
  const float2* stats;  // [B*rows] {rstd, -mean*rstd} or NULL
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  long long os_row;       // kRows / kSwiglu: output row stride (elements); rows of all batch items are consecutive
  long long rs_row;       // residual row stride
  long long plane_stride; // kPlanes: elements between planes
  int mode;
  int* status;
};

constexpr int kSmStages = 0;
constexpr int kSmSc = kStages * kStageBytes;  // 128 float2
constexpr int kSmBars = kSmSc + kTile * 8;
constexpr int kSmTotal = kSmBars + 128;
constexpr int kSmDynamic = kSmTotal + 1024;

enum Bar { FULL = 0, EMPTY = kStages, ACC_FULL = 2 * kStages, NUM_BARS = 2 * kStages + 1 };

__device__ __forceinline__ void stg256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

__device__ __forceinline__ float sigmoid_bf16(float x) {
  // the eager module applies sigmoid to the bf16 logits in place: round the logit, then the result
  const float xb = __bfloat162float(__float2bfloat16_rn(x));
  return 1.f / (1.f + __expf(-xb));
}

__global__ void __launch_bounds__(kThreads, 1)
linear_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w, const LinearParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kSmBars;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + kSmBars + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + kSmBars + NUM_BARS * 8 + 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tile_m = blockIdx.x % p.tiles_m;
  const int b = blockIdx.x / p.tiles_m;
  const int row0 = tile_m * kTile;
  const int n0 = blockIdx.y * kTile;
  const int steps = p.K / kStepK;

  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    abort_flag[1] = 0;
    for (int i = 0; i < kStages; ++i) {
      mbar_init(bars + (FULL + i) * 8, 1);
      mbar_init(bars + (EMPTY + i) * 8, 1);
    }
    mbar_init(bars + ACC_FULL * 8, 1);
    fence_mbar_init();
  }
  if (threadIdx.x < kTile) reinterpret_cast<float2*>(gen + kSmSc)[threadIdx.x] = p.sc[n0 + threadIdx.x];
  if (warp == 5) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_w);
      int issued = 0;
      for (int kk = 0; kk < steps; ++kk) {
        const int stage = kk % kStages;
        if (!mbar_wait(bars + (EMPTY + stage) * 8, ((kk / kStages) & 1) ^ 1, abort_flag)) break;
        const uint32_t full = bars + (FULL + stage) * 8;
        const uint32_t dst = base + kSmStages + stage * kStageBytes;
        mbar_expect_tx(full, kStageBytes);
        tma_load_4d(dst, &tm_a, full, (kk & 1) * kStepK, row0, kk >> 1, b);
        tma_load_2d(dst + kTile * kStepK * 2, &tm_w, full, kk * kStepK, n0);
        ++issued;
      }
      // If the loop was abandoned, give the copy still in flight a bounded chance to land.
      if (*abort_flag && issued > 0) {
        const int last = issued - 1;
        mbar_wait(bars + (FULL + last % kStages) * 8, (last / kStages) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(kTile, kTile);
      bool ok = true;
      for (int kk = 0; ok && kk < steps; ++kk) {
        const int stage = kk % kStages;
        ok = mbar_wait(bars + (FULL + stage) * 8, (kk / kStages) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a0 = base + kSmStages + stage * kStageBytes;
        const uint64_t da = make_smem_desc(a0, 16, 1024, kLayoutSw128);
        const uint64_t db = make_smem_desc(a0 + kTile * kStepK * 2, 16, 1024, kLayoutSw128);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_ss(tmem_base, da + k * 2, db + k * 2, idesc, (kk > 0 || k > 0) ? 1u : 0u);
        umma_commit(bars + (EMPTY + stage) * 8);
      }
      if (ok) umma_commit(bars + ACC_FULL * 8);
    }
  } else {
    const int m = warp * 32 + lane;
    const int row = row0 + m;
    const bool valid = row < p.rows;
    const long long grow = (long long)b * p.rows + row;
    float rstd = 1.f, nmr = 0.f;
    if (p.stats != nullptr && valid) {
      const float2 st = __ldg(p.stats + grow);
      rstd = st.x, nmr = st.y;
    }
    if (mbar_wait(bars + ACC_FULL * 8, 0, abort_flag)) {
      tc_fence_after();
      const float2* sc = reinterpret_cast<const float2*>(gen + kSmSc);
      const uint32_t lane_taddr = tmem_base + (uint32_t(warp * 32) << 16);
#pragma unroll 1
      for (int g = 0; g < 4; ++g) {
        uint32_t acc[32];
        tmem_ld32(lane_taddr + g * 32, acc);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const float2 t = sc[g * 32 + j];
          v[j] = fmaf(rstd, __uint_as_float(acc[j]), fmaf(nmr, t.x, t.y));
        }
        const int n = n0 + g * 32;
        if (!valid) continue;
        if (p.mode == kSwiglu) {
          uint32_t pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float g0 = v[16 + 2 * j], g1 = v[17 + 2 * j];
            pk[j] = pack_bf16x2(v[2 * j] * g0 / (1.f + __expf(-g0)), v[2 * j + 1] * g1 / (1.f + __expf(-g1)));
          }
          stg256(p.out + grow * p.os_row + (n >> 1), pk);
        } else {
          __nv_bfloat16* dst;
          if (p.mode == kPlanes) {
            const int which = n / (16 * 32), head = (n >> 5) & 15;
            dst = p.out + which * p.plane_stride + (((long long)b * 16 + head) * p.rows + row) * 32;
            if (which == 3) {
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = sigmoid_bf16(v[j]);
            }
          } else {
            dst = p.out + grow * p.os_row + n;
            if (p.residual != nullptr) {
              const uint4* r = reinterpret_cast<const uint4*>(p.residual + grow * p.rs_row + n);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const uint4 x = __ldg(r + c);
                const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                for (int t = 0; t < 4; ++t) v[c * 8 + 2 * t] += bf16_lo(w[t]), v[c * 8 + 2 * t + 1] += bf16_hi(w[t]);
              }
            }
          }
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(v[2 * j], v[2 * j + 1]);
          stg256(dst, pk);
          stg256(dst + 16, pk + 8);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 128);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

// {rstd, -mean * rstd} of every row: one warp per row, the row held in registers between the two passes.
__global__ void row_stats_kernel(const __nv_bfloat16* x, long long row_stride, long long rows, int K, float eps,
                                 float2* stats) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint32_t* src = reinterpret_cast<const uint32_t*>(x + row * row_stride);
  constexpr int kMaxPairs = 32;  // K <= 2048
  uint32_t v[kMaxPairs];
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPairs; ++i) {
    const int k2 = i * 32 + lane;  // index of a bf16 pair
    v[i] = 2 * k2 < K ? __ldg(src + k2) : 0u;
    sum += bf16_lo(v[i]) + bf16_hi(v[i]);
  }
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  const float mu = sum / float(K);
  float var = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxPairs; ++i) {
    if (2 * (i * 32 + lane) < K) {
      const float d0 = bf16_lo(v[i]) - mu, d1 = bf16_hi(v[i]) - mu;
      var = fmaf(d0, d0, fmaf(d1, d1, var));
    }
  }
  for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
  if (lane == 0) {
    const float rstd = rsqrtf(var / float(K) + eps);
    stats[row] = make_float2(rstd, -mu * rstd);
  }
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_row_stats(const void* x, int64_t row_stride, int64_t rows, int K, float eps, void* stats, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(x && stats, "row_stats: NULL pointer");
  B200TA_REQUIRE(rows > 0 && K > 0 && K <= 2048 && K % 2 == 0 && row_stride % 2 == 0,
                 "row_stats: need an even K <= 2048 and an even row stride (K=%d)", K);
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(x) & 3u) == 0, "row_stats: x must be 4-byte aligned");
  const int warps = 4;
  row_stats_kernel<<<unsigned((rows + warps - 1) / warps), warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), row_stride, rows, K, eps, static_cast<float2*>(stats));
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

int b200ta_linear(const void* a, int64_t as_b, int64_t as_row, int64_t as_chunk, const void* w, const void* sc,
                  const void* stats, const void* residual, int64_t rs_row, void* out, int64_t os_row,
                  int64_t plane_stride, int mode, int B, int rows, int K, int N, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(a && w && sc && out, "linear: NULL pointer");
  B200TA_REQUIRE(B > 0 && rows > 0 && K >= 128 && K % 128 == 0 && N >= 128 && N % 128 == 0,
                 "linear: K=%d and N=%d must be multiples of 128 (B=%d rows=%d)", K, N, B, rows);
  B200TA_REQUIRE(mode == kPlanes || mode == kRows || mode == kSwiglu, "linear: unknown mode %d", mode);
  B200TA_REQUIRE(mode != kPlanes || N == 4 * 16 * 32, "linear: the head-major form writes 4 planes of 16 heads x 32");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0 &&
                     as_row % 8 == 0 && as_chunk % 8 == 0 && (B == 1 || as_b % 8 == 0),
                 "linear: A and W must be 16-byte aligned with strides that are multiples of 8 elements");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(out) & 31u) == 0 && os_row % 16 == 0 && plane_stride % 16 == 0,
                 "linear: out must be 32-byte aligned with strides that are multiples of 16 elements");
  B200TA_REQUIRE(residual == nullptr || (mode == kRows && (reinterpret_cast<uintptr_t>(residual) & 15u) == 0 && rs_row % 8 == 0),
                 "linear: a residual needs the row form, 16-byte alignment and a row stride that is a multiple of 8");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  CUtensorMap tm_a, tm_w;
  {
    // element (b, row, k) of A at b*as_b + row*as_row + (k / 128)*as_chunk + k % 128
    uint64_t dims[4] = {128, uint64_t(rows), uint64_t(K / 128), uint64_t(B)};
    uint64_t strides[3] = {uint64_t(as_row) * 2, uint64_t(as_chunk) * 2, B == 1 ? 256u : uint64_t(as_b) * 2};
    uint32_t box[4] = {kStepK, kTile, 1, 1};
    rc = encode_tensor_map(&tm_a, a, 2, 4, dims, strides, box, SWZ_128, "linear A");
    if (rc != B200TA_OK) return rc;
  }
  {
    uint64_t dims[2] = {uint64_t(K), uint64_t(N)};
    uint64_t strides[1] = {uint64_t(K) * 2};
    uint32_t box[2] = {kStepK, kTile};
    rc = encode_tensor_map(&tm_w, w, 2, 2, dims, strides, box, SWZ_128, "linear W");
    if (rc != B200TA_OK) return rc;
  }
  LinearParams p{};
  p.B = B, p.rows = rows, p.K = K, p.N = N;
  p.tiles_m = (rows + kTile - 1) / kTile;
  p.sc = static_cast<const float2*>(sc);
  p.stats = static_cast<const float2*>(stats);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.os_row = os_row, p.rs_row = rs_row, p.plane_stride = plane_stride;
  p.mode = mode;
  p.status = st->status_dev;
  B200TA_CHECK_CUDA(cudaFuncSetAttribute(linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
  const dim3 grid(unsigned(B * p.tiles_m), unsigned(N / kTile));
  linear_kernel<<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_a, tm_w, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
