// Triangle-multiplication input stage for sm_100a:
//   x̂        = LayerNorm_in(z)
//   ab[ch]   = sigmoid(x̂·W_g[ch] + b_g) * (x̂·W_p[ch] + b_p) * mask          ch = a(0..127) | b(128..255)
// written channel-major, ab[b][ch][r][s], so that the contraction kernel finds the index it sums over (s)
// contiguous.  The incoming node calls this with the pair strides swapped (rows r = pair columns).
//
// The GEMM is computed transposed, D[channel, position] = W'[channel, :] · x̂[position, :]ᵀ: the folded weight
// rows are the A operand (M = 128 channels), the normalised tile of 128 positions the B operand (N = 128), so a
// TMEM lane is a channel and every epilogue thread owns one channel of 128 consecutive positions - exactly one
// contiguous 256-byte run of the channel-major output.  Per tile four such products: gate and value of the a
// channels (warpgroup 0 finishes them) and of the b channels (warpgroup 1).
//
// LayerNorm is folded into the weights (rows centred, per-row sum kept; gamma, beta and the biases included): the
// MMAs run on the raw tile as soon as it has landed, four statistics warps (one thread per position) compute mean
// and rstd of every position meanwhile, and the epilogue applies rstd[pos]·(D − mean[pos]·rowsum[ch]) + const[ch].
//
// Warp roles (704 threads): warps 0-15 epilogue - warpgroup g finishes the a (g < 2) or b (g >= 2) channels for
// the first (g even) or second (g odd) 64 positions of the tile -, warps 16-19 statistics, warp 20 TMA producer,
// warp 21 MMA issuer / TMEM owner.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kThreads = 704;
constexpr int kTileM = 128;                 // positions per tile
constexpr int kSmW = 0;                     // folded rows: 2 halves (64 channels of K each) x 512 rows x 128 B
constexpr int kWHalf = kTriInRows * 128;    // 64 KiB
constexpr int kSmZ = kSmW + 2 * kWHalf;     // 2 stages x 32 KiB
constexpr int kSmStats = kSmZ + 2 * 32768;  // 4 slots (tile i uses slot i & 3) x 3 x 128 floats: rstd, -mean*rstd, mask/2
constexpr int kStatsSlot = 3 * 512;
constexpr int kSmBars = kSmStats + 4 * kStatsSlot;
enum Bar { W_FULL = 0, Z_FULL = 1, STATS_READY = 3, Z_EMPTY = 7, ACC_FULL = 9, ACC_EMPTY = 11, NUM_BARS = 13 };
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

struct ProjectParams {
  int B, R, S;
  int tiles_s, num_tiles;
  const float2* sc;  // {rowsum, const} per folded row
  float eps;
  const float* mask;  // may be NULL
  long long ms_b, ms_r, ms_s;
  const float* b_scale;  // per batch item, multiplies the b channels; may be NULL
  __nv_bfloat16* ab;
  long long pitch;  // elements between rows of a plane
  int* status;
};

__device__ __forceinline__ void stg256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
trimul_project_kernel(const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_w,
                      const ProjectParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + kSmBars;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + kSmBars + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + kSmBars + NUM_BARS * 8 + 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    abort_flag[0] = 0, abort_flag[1] = 0;
    mbar_init(bars + W_FULL * 8, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + (Z_FULL + i) * 8, 1);
      mbar_init(bars + (Z_EMPTY + i) * 8, 5);   // the MMA commit + the four statistics warps have read the tile
      mbar_init(bars + (ACC_FULL + i) * 8, 1);  // per warpgroup
      mbar_init(bars + (ACC_EMPTY + i) * 8, 8);  // two warpgroups read each accumulator pair
    }
    // statistics of a tile written (the four statistics warps): one barrier per statistics slot, because the
    // statistics of tile t + 2 may be complete before the epilogue of tile t has looked at its barrier
    for (int i = 0; i < 4; ++i) mbar_init(bars + (STATS_READY + i) * 8, 4);
    fence_mbar_init();
  }
  if (warp == 21) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int my_tiles = (p.num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;

  if (warp == 20) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_z);
      tma_prefetch_desc(&tm_w);
      mbar_expect_tx(bars + W_FULL * 8, 2 * kWHalf);
      for (int kh = 0; kh < 2; ++kh)
        for (int j = 0; j < kTriInRows / 128; ++j)
          tma_load_2d(base + kSmW + kh * kWHalf + j * 128 * 128, &tm_w, bars + W_FULL * 8, kh * 64, j * 128);
      int issued = 0;
      for (int i = 0; i < my_tiles; ++i) {
        const int tile = blockIdx.x + i * gridDim.x;
        const int st = tile % p.tiles_s, br = tile / p.tiles_s;
        const int r = br % p.R, b = br / p.R;
        const int stage = i & 1;
        if (!mbar_wait(bars + (Z_EMPTY + stage) * 8, ((i >> 1) & 1) ^ 1, abort_flag)) break;
        const uint32_t full = bars + (Z_FULL + stage) * 8;
        mbar_expect_tx(full, 32768);
        tma_load_4d(base + kSmZ + stage * 32768, &tm_z, full, 0, st * kTileM, r, b);
        tma_load_4d(base + kSmZ + stage * 32768 + 16384, &tm_z, full, 64, st * kTileM, r, b);
        ++issued;
      }
      if (*abort_flag && issued > 0) {
        const int last = issued - 1;
        mbar_wait(bars + (Z_FULL + (last & 1)) * 8, (last >> 1) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 21) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, kTileM);
      bool ok = mbar_wait(bars + W_FULL * 8, 0, abort_flag);
      for (int i = 0; ok && i < my_tiles; ++i) {
        const int stage = i & 1;
        ok = mbar_wait(bars + (Z_FULL + stage) * 8, (i >> 1) & 1, abort_flag);
        if (!ok) break;
        const uint64_t dz = make_smem_desc(base + kSmZ + stage * 32768, 16, 1024, kLayoutSw128);
        for (int wg = 0; ok && wg < 2; ++wg) {
          ok = mbar_wait(bars + (ACC_EMPTY + wg) * 8, (i & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int acc = 0; acc < 2; ++acc) {  // gate rows, then value rows of this warpgroup's channels
            const uint32_t d = tmem_base + (wg * 2 + acc) * 128;
            const uint64_t dw = make_smem_desc(base + kSmW + (wg * 2 + acc) * 128 * 128, 16, 1024, kLayoutSw128);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              umma_ss(d, dw + ((k >> 2) * (kWHalf >> 4) + (k & 3) * 2), dz + ((k >> 2) * (16384 >> 4) + (k & 3) * 2), idesc,
                      k > 0 ? 1u : 0u);
          }
          umma_commit(bars + (ACC_FULL + wg) * 8);
        }
        if (!ok) break;
        umma_commit(bars + (Z_EMPTY + stage) * 8);
      }
    }
  } else if (warp >= 16 && warp < 20) {
    // ------------------------------------------------------------------ statistics: one thread per position
    const int m = (warp - 16) * 32 + lane;
    bool ok = true;
    for (int i = 0; ok && i < my_tiles; ++i) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int st = tile % p.tiles_s, br = tile / p.tiles_s;
      const int r = br % p.R, b = br / p.R;
      const int stage = i & 1;
      const int s = st * kTileM + m;
      float mval = 0.f;
      if (s < p.S) mval = p.mask ? __ldg(p.mask + b * p.ms_b + r * p.ms_r + (long long)s * p.ms_s) : 1.f;
      ok = mbar_wait(bars + (Z_FULL + stage) * 8, (i >> 1) & 1, abort_flag);
      if (!ok) break;
      const uint32_t z0 = base + kSmZ + stage * 32768;
      // two passes over the 256-byte row in shared memory (mean, then squared deviations), eight 16-byte loads in
      // flight at a time; the reads are conflict-free and nothing is written back
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int c = 0; c < 16; ++c) {
        const uint4 x = lds128(z0 + (c >> 3) * 16384 + sw128_offset(m, c & 7));
        sum4[0] += bf16_lo(x.x) + bf16_hi(x.x);
        sum4[1] += bf16_lo(x.y) + bf16_hi(x.y);
        sum4[2] += bf16_lo(x.z) + bf16_hi(x.z);
        sum4[3] += bf16_lo(x.w) + bf16_hi(x.w);
      }
      const float mu = ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3])) * (1.f / kC);
      float var4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
      for (int c = 0; c < 16; ++c) {
        const uint4 x = lds128(z0 + (c >> 3) * 16384 + sw128_offset(m, c & 7));
        const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float d0 = bf16_lo(w4[e]) - mu, d1 = bf16_hi(w4[e]) - mu;
          var4[e] = fmaf(d0, d0, var4[e]);
          var4[e] = fmaf(d1, d1, var4[e]);
        }
      }
      const float rstd = rsqrtf(((var4[0] + var4[1]) + (var4[2] + var4[3])) * (1.f / kC) + p.eps);
      // Statistics and mask go to one of four slots: the epilogue of a tile reads its slot while the statistics of
      // the next two tiles are written.  A slot is rewritten four tiles later, when that epilogue is long done
      // (the MMAs of tile t + 1 wait for the accumulators of tile t, the loads of tile t + 3 for those MMAs).
      float* slot = reinterpret_cast<float*>(gen + kSmStats + (i & 3) * kStatsSlot);
      slot[m] = rstd;
      slot[128 + m] = -mu * rstd;
      slot[256 + m] = 0.5f * mval;  // sigmoid(g) * v * mask = tanh(g/2) * h + h with h = v * mask / 2
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bars + (STATS_READY + (i & 3)) * 8);
        mbar_arrive(bars + (Z_EMPTY + stage) * 8);  // done reading the tile
      }
    }
  } else if (warp < 16) {
    // ------------------------------------------------------------------ epilogue warps: one thread per channel
    const int wg = warp >> 3;        // 0: a channels, 1: b channels
    const int half = (warp >> 2) & 1;  // which 64 positions of the tile
    const int ch = (warp & 3) * 32 + lane;  // channel inside the 128 == TMEM lane
    // gate columns of these 64 positions; the value columns lie 128 further
    const uint32_t acc = tmem_base + (uint32_t((warp & 3) * 32) << 16) + wg * 256 + half * 64;
    const float2 kg = p.sc[wg * 256 + ch], kp = p.sc[wg * 256 + 128 + ch];  // {rowsum, const} of the gate / value row
    const uint64_t cg2 = pack_f32x2(kg.y, kg.y), cp2 = pack_f32x2(kp.y, kp.y);
    const uint64_t rg2 = pack_f32x2(kg.x, kg.x), rp2 = pack_f32x2(kp.x, kp.x);
    bool ok = true;
    for (int i = 0; ok && i < my_tiles; ++i) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int st = tile % p.tiles_s, br = tile / p.tiles_s;
      const int r = br % p.R, b = br / p.R;
      const float bscale = (wg == 1 && p.b_scale) ? __ldg(p.b_scale + b) : 1.f;
      const uint64_t hs2 = pack_f32x2(bscale, bscale);
      // per position: rstd, -mean*rstd, mask/2, as pairs of neighbouring positions
      const float2* stats = reinterpret_cast<const float2*>(gen + kSmStats + (i & 3) * kStatsSlot) + half * 32;
      __nv_bfloat16* dst = p.ab + ((long long)(b * 2 + wg) * kTriHidden + ch) * p.R * p.pitch + (long long)r * p.pitch +
                           st * kTileM + half * 64;
      ok = mbar_wait(bars + (STATS_READY + (i & 3)) * 8, (i >> 2) & 1, abort_flag) &&
           mbar_wait(bars + (ACC_FULL + wg) * 8, i & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      // 8 positions at a time; the TMEM loads of the next chunk are in flight while this one is computed
      uint32_t g[2][8], v[2][8];
      tmem_ld8(acc, g[0]);
      tmem_ld8(acc + 128, v[0]);
      uint32_t packed[8];
#pragma unroll
      for (int part = 0; part < 8; ++part) {
        tmem_ld_wait();
        if (part + 1 < 8) {
          tmem_ld8(acc + (part + 1) * 8, g[(part + 1) & 1]);
          tmem_ld8(acc + 128 + (part + 1) * 8, v[(part + 1) & 1]);
        }
        const uint32_t (&gg)[8] = g[part & 1];
        const uint32_t (&vv)[8] = v[part & 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // packed fp32x2 math on two positions: LayerNorm finished per position, gate rows are pre-halved
          const float2 rs = stats[part * 4 + j], nm = stats[64 + part * 4 + j], mh = stats[128 + part * 4 + j];
          const uint64_t rs2 = pack_f32x2(rs.x, rs.y), nm2 = pack_f32x2(nm.x, nm.y);
          float a0, a1;
          unpack_f32x2(fma_f32x2(rs2, pack_f32x2(__uint_as_float(gg[2 * j]), __uint_as_float(gg[2 * j + 1])),
                                 fma_f32x2(nm2, rg2, cg2)), a0, a1);
          const uint64_t val2 = fma_f32x2(rs2, pack_f32x2(__uint_as_float(vv[2 * j]), __uint_as_float(vv[2 * j + 1])),
                                          fma_f32x2(nm2, rp2, cp2));
          // sigmoid(g) * v * mask = tanh(g/2) * h + h with h = v * mask / 2
          const uint64_t h2 = mul_f32x2(val2, mul_f32x2(pack_f32x2(mh.x, mh.y), hs2));
          float o0, o1;
          unpack_f32x2(fma_f32x2(pack_f32x2(tanh_approx(a0), tanh_approx(a1)), h2, h2), o0, o1);
          packed[(part & 1) * 4 + j] = pack_bf16x2(o0, o1);
        }
        if ((part & 1) && st * kTileM + half * 64 + (part - 1) * 8 + 16 <= p.pitch) stg256(dst + (part - 1) * 8, packed);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (ACC_EMPTY + wg) * 8);
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 21) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_trimul_project(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const float* mask, int64_t ms_b,
                          int64_t ms_r, int64_t ms_s, const float* b_scale, const void* packed, float eps, void* ab,
                          int64_t pitch, int B, int R, int S, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(z && packed && ab, "trimul_project: NULL pointer");
  B200TA_REQUIRE(B > 0 && R > 0 && S > 0, "trimul_project: bad sizes B=%d R=%d S=%d", B, R, S);
  B200TA_REQUIRE(pitch >= S && pitch % 16 == 0, "trimul_project: pitch=%lld must be a multiple of 16 and >= S=%d",
                 (long long)pitch, S);
  B200TA_REQUIRE(zs_b % 8 == 0 && zs_r % 8 == 0 && zs_s % 8 == 0 && zs_b >= 0 && zs_r >= 0 && zs_s >= 0,
                 "trimul_project: z element strides must be non-negative multiples of 8 (16 bytes)");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "trimul_project: packed must be 256-byte aligned");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(ab) & 31u) == 0, "trimul_project: ab must be 32-byte aligned");
  B200TA_REQUIRE(int64_t(B) * R < (int64_t(1) << 31), "trimul_project: B*R too large");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  CUtensorMap tm_z, tm_w;
  {
    // (c, s, r, b); a size-1 dimension may carry any stride: give it a valid one
    auto fix = [](int64_t stride, int extent) -> uint64_t { return extent == 1 ? 256u : uint64_t(stride) * 2u; };
    uint64_t dims[4] = {uint64_t(kC), uint64_t(S), uint64_t(R), uint64_t(B)};
    uint64_t strides[3] = {fix(zs_s, S), fix(zs_r, R), fix(zs_b, B)};
    uint32_t box[4] = {64, kTileM, 1, 1};
    rc = encode_tensor_map(&tm_z, z, 2, 4, dims, strides, box, SWZ_128, "trimul_project z");
    if (rc != B200TA_OK) return rc;
  }
  const char* pk = static_cast<const char*>(packed);
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(kTriRows)};
    uint64_t strides[1] = {uint64_t(kC) * 2};
    uint32_t box[2] = {64, 128};
    rc = encode_tensor_map(&tm_w, pk + kTriWOff, 2, 2, dims, strides, box, SWZ_128, "trimul_project weights");
    if (rc != B200TA_OK) return rc;
  }
  ProjectParams p{};
  p.B = B, p.R = R, p.S = S;
  p.tiles_s = (S + kTileM - 1) / kTileM;
  p.num_tiles = B * R * p.tiles_s;
  p.sc = reinterpret_cast<const float2*>(pk + kTriScOff);
  p.eps = eps;
  p.mask = mask;
  p.ms_b = ms_b, p.ms_r = ms_r, p.ms_s = ms_s;
  p.b_scale = b_scale;
  p.ab = static_cast<__nv_bfloat16*>(ab);
  p.pitch = pitch;
  p.status = st->status_dev;

  B200TA_CHECK_CUDA(cudaFuncSetAttribute(trimul_project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  trimul_project_kernel<<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_z, tm_w, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
