// Triangle-multiplication output stage for sm_100a:
//   out[b,i,j,:] = sigmoid(LN_in(z[b,i,j,:])·W_goᵀ + b_go) ⊙ (LN_out(x[b,:,i,j])·W_poᵀ + b_po)   [+ z]   [* mask]
// x is the contraction result, channel-major x[b][d][i][j] (bf16).  One tile = 128 consecutive positions j of one
// pair row (b, i); per tile two tcgen05 GEMMs share one accumulator slot (256 TMEM columns, double-buffered):
//   D_g[pos, ch] = z[pos, :] · W_go'[ch, :]ᵀ    A = the raw z tile (K-major)
//   D_p[pos, ch] = x[:, pos]ᵀ · W_po'[ch, :]ᵀ   A = the x tile as it lies in memory, [d][pos] = MN-major
// Both LayerNorms are folded into the weights (rows centred, per-row sum kept): the epilogue, one thread per
// position, applies rstd·(D − mean·rowsum) + const with the statistics the statistics warps computed from the two
// tiles while the MMAs ran - neither tile is rewritten and the MMAs wait for nothing but the loads.
//
// Warp roles (448 threads): warps 0-7 epilogue (thread = position; the two warpgroups take alternate groups of 32
// output channels), warps 8-11 statistics (z rows: one thread per position; x columns: a thread takes two
// neighbouring positions over half of the channels), warp 12 TMA producer, warp 13 MMA issuer / TMEM owner.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kThreads = 448;
constexpr int kTileM = 128;
constexpr int kSmW = 0;                      // W_go' and W_po': 2 matrices x 2 K-halves x 128 rows x 128 B
constexpr int kSmZ = kSmW + 65536;           // 2 stages x 32 KiB
constexpr int kSmX = kSmZ + 2 * 32768;       // 2 stages x 32 KiB
constexpr int kSmConst = kSmX + 2 * 32768;   // per channel pair: float4 [64] {c_gate0, c_gate1, rowsum_g0, rowsum_g1}, float4 [64] {c_p0, c_p1, rowsum_p0, rowsum_p1}
constexpr int kSmStats = kSmConst + 2048;    // 4 slots (tile i uses slot i & 3) x { float4 [128] {rstd_o, -mean_o*rstd_o, rstd_i, -mean_i*rstd_i}, float [128] mask }
constexpr int kStatsSlot = 2048 + 512;
constexpr int kSmXch = kSmStats + 4 * kStatsSlot;  // 2 x float4 [128] partial x statistics (alternating per tile)
constexpr int kSmBars = kSmXch + 2 * 2048;
enum Bar { W_FULL = 0, IN_FULL = 1, READY = 3, IN_EMPTY = 7, ACC_FULL = 9, ACC_EMPTY = 11, XCH = 13, NUM_BARS = 14 };
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

struct OutputParams {
  int B, N;  // pair tensor [B, N, N, 128]
  int tiles_j, num_tiles;
  const float2* sc;  // folded {rowsum, const} of the output gate rows, then of the output projection rows
  float eps;
  const __nv_bfloat16* z;  // residual source (same tensor the z tiles are loaded from)
  long long zs_b, zs_i, zs_j;
  int add_residual;
  const float* mask;  // [B, N, N] via strides; NULL = no output mask
  long long ms_b, ms_i, ms_j;
  __nv_bfloat16* out;
  long long os_b, os_i, os_j;
  int* status;
};

__device__ __forceinline__ void stg256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__global__ void __launch_bounds__(kThreads, 1)
trimul_output_kernel(const __grid_constant__ CUtensorMap tm_z, const __grid_constant__ CUtensorMap tm_x,
                     const __grid_constant__ CUtensorMap tm_w, const OutputParams p) {
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
    mbar_init(bars + XCH * 8, 4);
    // statistics written (the four statistics warps): one barrier per statistics slot, because the statistics of
    // tile t + 2 may be complete before the epilogue of tile t has looked at its barrier
    for (int i = 0; i < 4; ++i) mbar_init(bars + (READY + i) * 8, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + (IN_FULL + i) * 8, 1);
      mbar_init(bars + (IN_EMPTY + i) * 8, 5);  // the MMA commit + the four statistics warps have read the tiles
      mbar_init(bars + (ACC_FULL + i) * 8, 1);
      mbar_init(bars + (ACC_EMPTY + i) * 8, 8);
    }
    fence_mbar_init();
  }
  // per-channel constants of the epilogue
  if (threadIdx.x < kC / 2) {
    const int c = 2 * threadIdx.x;
    const float2 g0 = p.sc[c], g1 = p.sc[c + 1], q0 = p.sc[kC + c], q1 = p.sc[kC + c + 1];
    reinterpret_cast<float4*>(gen + kSmConst)[threadIdx.x] = make_float4(g0.y, g1.y, g0.x, g1.x);
    reinterpret_cast<float4*>(gen + kSmConst + 1024)[threadIdx.x] = make_float4(q0.y, q1.y, q0.x, q1.x);
  }
  if (warp == 13) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int my_tiles = (p.num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;

  if (warp == 12) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_z);
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w);
      mbar_expect_tx(bars + W_FULL * 8, 65536);
      for (int mat = 0; mat < 2; ++mat)
        for (int kh = 0; kh < 2; ++kh)
          tma_load_2d(base + kSmW + mat * 32768 + kh * 16384, &tm_w, bars + W_FULL * 8, kh * 64, kTriInRows + mat * kC);
      int issued = 0;
      for (int it = 0; it < my_tiles; ++it) {
        const int tile = blockIdx.x + it * gridDim.x;
        const int jt = tile % p.tiles_j, bi = tile / p.tiles_j;
        const int i = bi % p.N, b = bi / p.N;
        const int stage = it & 1;
        if (!mbar_wait(bars + (IN_EMPTY + stage) * 8, ((it >> 1) & 1) ^ 1, abort_flag)) break;
        const uint32_t full = bars + (IN_FULL + stage) * 8;
        mbar_expect_tx(full, 65536);
        tma_load_4d(base + kSmZ + stage * 32768, &tm_z, full, 0, jt * kTileM, i, b);
        tma_load_4d(base + kSmZ + stage * 32768 + 16384, &tm_z, full, 64, jt * kTileM, i, b);
        tma_load_3d(base + kSmX + stage * 32768, &tm_x, full, jt * kTileM, i, b * kTriHidden);
        tma_load_3d(base + kSmX + stage * 32768 + 16384, &tm_x, full, jt * kTileM + 64, i, b * kTriHidden);
        ++issued;
      }
      if (*abort_flag && issued > 0) {
        const int last = issued - 1;
        mbar_wait(bars + (IN_FULL + (last & 1)) * 8, (last >> 1) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 13) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_g = make_idesc_bf16(kTileM, kC);              // both operands K-major
      constexpr uint32_t idesc_p = make_idesc_bf16(kTileM, kC, true, false);  // A (the x tile) MN-major
      bool ok = mbar_wait(bars + W_FULL * 8, 0, abort_flag);
      for (int it = 0; ok && it < my_tiles; ++it) {
        const int stage = it & 1, slot = it & 1;
        ok = mbar_wait(bars + (IN_FULL + stage) * 8, (it >> 1) & 1, abort_flag);
        ok = ok && mbar_wait(bars + (ACC_EMPTY + slot) * 8, ((it >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem_base + slot * 256;
        const uint64_t dz = make_smem_desc(base + kSmZ + stage * 32768, 16, 1024, kLayoutSw128);
        const uint64_t dwg = make_smem_desc(base + kSmW, 16, 1024, kLayoutSw128);
        const uint64_t dwp = make_smem_desc(base + kSmW + 32768, 16, 1024, kLayoutSw128);
        // x tile: [128 d][64 j] blocks of 128-byte rows, the two 64-position blocks 16 KiB apart; as A[pos][d] this
        // is MN-major, a K step of 16 channels is 16 rows = 2 KiB
        const uint64_t dx = make_smem_desc(base + kSmX + stage * 32768, 16384, 1024, kLayoutSw128);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t koff = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
          umma_ss(d, dz + koff, dwg + koff, idesc_g, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_ss(d + 128, dx + k * 128, dwp + ((k >> 2) * (16384 >> 4) + (k & 3) * 2), idesc_p, k > 0 ? 1u : 0u);
        umma_commit(bars + (ACC_FULL + slot) * 8);
        umma_commit(bars + (IN_EMPTY + stage) * 8);
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ normaliser
    const int t = (warp - 8) * 32 + lane;
    bool ok = true;
    for (int it = 0; ok && it < my_tiles; ++it) {
      const int tile = blockIdx.x + it * gridDim.x;
      const int jt = tile % p.tiles_j, bi = tile / p.tiles_j;
      const int i = bi % p.N, b = bi / p.N;
      const int stage = it & 1;
      const int j = jt * kTileM + t;
      float mval = 1.f;
      if (p.mask != nullptr) mval = j < p.N ? __ldg(p.mask + b * p.ms_b + i * p.ms_i + (long long)j * p.ms_j) : 0.f;
      ok = mbar_wait(bars + (IN_FULL + stage) * 8, (it >> 1) & 1, abort_flag);
      if (!ok) break;
      // ---- z row t: mean and variance (two passes over the row in shared memory; nothing is written back)
      float rstd_i, nmr_i;
      {
        const uint32_t z0 = base + kSmZ + stage * 32768;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int c = 0; c < 16; ++c) {
          const uint4 x = lds128(z0 + (c >> 3) * 16384 + sw128_offset(t, c & 7));
          sum4[0] += bf16_lo(x.x) + bf16_hi(x.x);
          sum4[1] += bf16_lo(x.y) + bf16_hi(x.y);
          sum4[2] += bf16_lo(x.z) + bf16_hi(x.z);
          sum4[3] += bf16_lo(x.w) + bf16_hi(x.w);
        }
        const float mu = ((sum4[0] + sum4[1]) + (sum4[2] + sum4[3])) * (1.f / kC);
        float var4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 8
        for (int c = 0; c < 16; ++c) {
          const uint4 x = lds128(z0 + (c >> 3) * 16384 + sw128_offset(t, c & 7));
          const uint32_t w4[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float d0 = bf16_lo(w4[e]) - mu, d1 = bf16_hi(w4[e]) - mu;
            var4[e] = fmaf(d0, d0, var4[e]);
            var4[e] = fmaf(d1, d1, var4[e]);
          }
        }
        rstd_i = rsqrtf(((var4[0] + var4[1]) + (var4[2] + var4[3])) * (1.f / kC) + p.eps);
        nmr_i = -mu * rstd_i;
      }
      // ---- x columns: this thread takes positions 2q, 2q+1 over channels [64 h, 64 h + 64)
      {
        const int q = t & 63, h = t >> 6;
        const int jj = (2 * q) & 63;
        const uint32_t x0 = base + kSmX + stage * 32768 + ((2 * q) >> 6) * 16384 + (jj & 7) * 2;
        const uint32_t chunk = uint32_t(jj >> 3);
        uint32_t w[64];
#pragma unroll
        for (int d = 0; d < 64; ++d) {
          const uint32_t row = uint32_t(h * 64 + d);
          w[d] = lds32(x0 + row * 128 + ((chunk ^ (row & 7)) << 4));
        }
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int d = 0; d < 64; ++d) s0 += bf16_lo(w[d]), s1 += bf16_hi(w[d]);
        const float m0 = s0 * (1.f / 64), m1 = s1 * (1.f / 64);
        float q0 = 0.f, q1 = 0.f;
#pragma unroll
        for (int d = 0; d < 64; ++d) {
          const float d0 = bf16_lo(w[d]) - m0, d1 = bf16_hi(w[d]) - m1;
          q0 = fmaf(d0, d0, q0), q1 = fmaf(d1, d1, q1);
        }
        reinterpret_cast<float4*>(gen + kSmXch + (it & 1) * 2048)[t] = make_float4(m0, q0, m1, q1);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + XCH * 8);
      ok = mbar_wait(bars + XCH * 8, it & 1, abort_flag);
      if (!ok) break;
      {
        // position t = 2q + e: combine the two channel halves (means m, sums of squared deviations Q of 64 each)
        const int q = t >> 1, e = t & 1;
        const float4 a = reinterpret_cast<const float4*>(gen + kSmXch + (it & 1) * 2048)[q];
        const float4 c = reinterpret_cast<const float4*>(gen + kSmXch + (it & 1) * 2048)[64 + q];
        const float ma = e ? a.z : a.x, qa = e ? a.w : a.y, mc = e ? c.z : c.x, qc = e ? c.w : c.y;
        const float mean = 0.5f * (ma + mc);
        const float var = (qa + qc + (ma - mc) * (ma - mc) * 32.f) * (1.f / kTriHidden);
        const float rstd = rsqrtf(var + p.eps);
        // Statistics and mask go to one of four slots: the epilogue of a tile may still read its slot while the
        // next two tiles' statistics are written (the stage itself is handed back below, before the epilogue ran).
        uint8_t* slot = gen + kSmStats + (it & 3) * kStatsSlot;
        reinterpret_cast<float4*>(slot)[t] = make_float4(rstd, -mean * rstd, rstd_i, nmr_i);
        reinterpret_cast<float*>(slot + 2048)[t] = mval;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(bars + (READY + (it & 3)) * 8);
        mbar_arrive(bars + (IN_EMPTY + stage) * 8);  // done reading the two tiles
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps: one thread per position
    const int e = warp >> 2;
    const int m = (warp & 3) * 32 + lane;
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const float4* c4 = reinterpret_cast<const float4*>(gen + kSmConst);         // per channel pair
    const float4* c4b = reinterpret_cast<const float4*>(gen + kSmConst + 1024);  // per channel pair
    bool ok = true;
    for (int it = 0; ok && it < my_tiles; ++it) {
      const int tile = blockIdx.x + it * gridDim.x;
      const int jt = tile % p.tiles_j, bi = tile / p.tiles_j;
      const int i = bi % p.N, b = bi / p.N;
      const int slot = it & 1;
      const int j = jt * kTileM + m;
      // The residual values do not depend on the accumulators: fetch this thread's 2 x 32 channels (they were just
      // loaded as part of the z tile, so they come from L2) before waiting for the MMAs.
      uint32_t res[2][16];
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        if (p.add_residual && j < p.N) {
          const uint4* rp = reinterpret_cast<const uint4*>(p.z + b * p.zs_b + i * p.zs_i + (long long)j * p.zs_j +
                                                           (e + 2 * gi) * 32);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 x = __ldg(rp + c);
            res[gi][c * 4 + 0] = x.x, res[gi][c * 4 + 1] = x.y, res[gi][c * 4 + 2] = x.z, res[gi][c * 4 + 3] = x.w;
          }
        } else {
#pragma unroll
          for (int c = 0; c < 16; ++c) res[gi][c] = 0u;
        }
      }
      ok = mbar_wait(bars + (READY + (it & 3)) * 8, (it >> 2) & 1, abort_flag) &&
           mbar_wait(bars + (ACC_FULL + slot) * 8, (it >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      const uint8_t* stats = gen + kSmStats + (it & 3) * kStatsSlot;
      const float4 stv = reinterpret_cast<const float4*>(stats)[m];
      const float mval = reinterpret_cast<const float*>(stats + 2048)[m];
      const uint64_t rstd2 = pack_f32x2(stv.x, stv.x), nmr2 = pack_f32x2(stv.y, stv.y), mval2 = pack_f32x2(mval, mval);
      const uint64_t rstdg2 = pack_f32x2(stv.z, stv.z), nmrg2 = pack_f32x2(stv.w, stv.w);
      const uint64_t half2 = pack_f32x2(0.5f, 0.5f);
      // four chunks of 16 output channels: [32 g + 16 h, +16) for this warpgroup's groups g = e, e + 2; the TMEM
      // loads of the next chunk are in flight while this one is computed
      uint32_t ag[2][16], ap[2][16];
      const uint32_t acc = lane_taddr + slot * 256;
      tmem_ld16(acc + e * 32, ag[0]);
      tmem_ld16(acc + 128 + e * 32, ap[0]);
#pragma unroll
      for (int ck = 0; ck < 4; ++ck) {
        const int g = e + 2 * (ck >> 1), h = ck & 1;
        const int ch0 = g * 32 + h * 16;
        tmem_ld_wait();
        if (ck + 1 < 4) {
          const int gn = e + 2 * ((ck + 1) >> 1), hn = (ck + 1) & 1;
          tmem_ld16(acc + gn * 32 + hn * 16, ag[(ck + 1) & 1]);
          tmem_ld16(acc + 128 + gn * 32 + hn * 16, ap[(ck + 1) & 1]);
        }
        const uint32_t (&xg)[16] = ag[ck & 1];
        const uint32_t (&xp)[16] = ap[ck & 1];
        uint32_t packed[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          // two channels at a time, packed fp32x2 math; constants per channel pair: {const0, const1, rowsum0,
          // rowsum1} of the gate rows and of the projection rows
          const float4 ka = c4[(ch0 >> 1) + c];
          const float4 kb = c4b[(ch0 >> 1) + c];
          float a0, a1;
          unpack_f32x2(fma_f32x2(rstdg2, pack_f32x2(__uint_as_float(xg[2 * c]), __uint_as_float(xg[2 * c + 1])),
                                 fma_f32x2(nmrg2, pack_f32x2(ka.z, ka.w), pack_f32x2(ka.x, ka.y))),
                       a0, a1);
          // gate rows are pre-halved: sigmoid(x) = 0.5 * tanh(x / 2) + 0.5
          const uint64_t s2 = fma_f32x2(pack_f32x2(tanh_approx(a0), tanh_approx(a1)), half2, half2);
          const uint64_t v2 = fma_f32x2(rstd2, pack_f32x2(__uint_as_float(xp[2 * c]), __uint_as_float(xp[2 * c + 1])),
                                        fma_f32x2(nmr2, pack_f32x2(kb.z, kb.w), pack_f32x2(kb.x, kb.y)));
          const uint32_t r = res[ck >> 1][h * 8 + c];
          float o0, o1;
          unpack_f32x2(mul_f32x2(fma_f32x2(s2, v2, pack_f32x2(bf16_lo(r), bf16_hi(r))), mval2), o0, o1);
          packed[c] = pack_bf16x2(o0, o1);
        }
        if (j < p.N) stg256(p.out + b * p.os_b + i * p.os_i + (long long)j * p.os_j + ch0, packed);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (ACC_EMPTY + slot) * 8);
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 13) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_trimul_output(const void* z, int64_t zs_b, int64_t zs_i, int64_t zs_j, const void* x, int64_t pitch,
                         const float* mask, int64_t ms_b, int64_t ms_i, int64_t ms_j, const void* packed, float eps,
                         int add_residual, void* out, int64_t os_b, int64_t os_i, int64_t os_j, int B, int N,
                         void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(z && x && packed && out, "trimul_output: NULL pointer");
  B200TA_REQUIRE(B > 0 && N > 0, "trimul_output: bad sizes B=%d N=%d", B, N);
  B200TA_REQUIRE(pitch >= N && pitch % 16 == 0, "trimul_output: pitch=%lld must be a multiple of 16 and >= N=%d",
                 (long long)pitch, N);
  for (int64_t s : {zs_b, zs_i, zs_j, os_b, os_i, os_j})
    B200TA_REQUIRE(s >= 0 && s % 16 == 0, "trimul_output: z/out element strides must be non-negative multiples of 16");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "trimul_output: packed must be 256-byte aligned");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(z) & 31u) == 0 && (reinterpret_cast<uintptr_t>(out) & 31u) == 0 &&
                     (reinterpret_cast<uintptr_t>(x) & 31u) == 0,
                 "trimul_output: z, x and out must be 32-byte aligned");
  B200TA_REQUIRE(int64_t(B) * N < (int64_t(1) << 31), "trimul_output: B*N too large");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  CUtensorMap tm_z, tm_x, tm_w;
  {
    auto fix = [](int64_t stride, int extent) -> uint64_t { return extent == 1 ? 256u : uint64_t(stride) * 2u; };
    uint64_t dims[4] = {uint64_t(kC), uint64_t(N), uint64_t(N), uint64_t(B)};
    uint64_t strides[3] = {fix(zs_j, N), fix(zs_i, N), fix(zs_b, B)};
    uint32_t box[4] = {64, kTileM, 1, 1};
    rc = encode_tensor_map(&tm_z, z, 2, 4, dims, strides, box, SWZ_128, "trimul_output z");
    if (rc != B200TA_OK) return rc;
  }
  {
    // (j, i, plane): one load = 64 positions x 128 channels of one pair row
    uint64_t dims[3] = {uint64_t(N), uint64_t(N), uint64_t(B) * kTriHidden};
    uint64_t strides[2] = {uint64_t(pitch) * 2, uint64_t(pitch) * N * 2};
    uint32_t box[3] = {64, 1, kTriHidden};
    rc = encode_tensor_map(&tm_x, x, 2, 3, dims, strides, box, SWZ_128, "trimul_output x");
    if (rc != B200TA_OK) return rc;
  }
  const char* pk = static_cast<const char*>(packed);
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(kTriRows)};
    uint64_t strides[1] = {uint64_t(kC) * 2};
    uint32_t box[2] = {64, 128};
    rc = encode_tensor_map(&tm_w, pk + kTriWOff, 2, 2, dims, strides, box, SWZ_128, "trimul_output weights");
    if (rc != B200TA_OK) return rc;
  }
  OutputParams p{};
  p.B = B, p.N = N;
  p.tiles_j = (N + kTileM - 1) / kTileM;
  p.num_tiles = B * N * p.tiles_j;
  p.sc = reinterpret_cast<const float2*>(pk + kTriScOff) + kTriInRows;
  p.eps = eps;
  p.z = static_cast<const __nv_bfloat16*>(z);
  p.zs_b = zs_b, p.zs_i = zs_i, p.zs_j = zs_j;
  p.add_residual = add_residual ? 1 : 0;
  p.mask = mask;
  p.ms_b = ms_b, p.ms_i = ms_i, p.ms_j = ms_j;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.os_b = os_b, p.os_i = os_i, p.os_j = os_j;
  p.status = st->status_dev;

  B200TA_CHECK_CUDA(cudaFuncSetAttribute(trimul_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  trimul_output_kernel<<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_z, tm_x, tm_w, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
