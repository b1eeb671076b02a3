// Pair transition for sm_100a: out = [x +] mask * ( (silu(gate) * value) · W2ᵀ ),
// [value|gate] = LayerNorm(x) · W1ᵀ, hidden 512, one kernel, hidden kept on chip.
// The ReLU form (kRelu) computes out = [x +] mask * ( relu(LayerNorm(x) · W1ᵀ + b1) · W2ᵀ + b2 ) with the same
// pipeline: its 512 hidden rows sit in the value half of the packed first linear, the gate half is zero.
//
// A persistent CTA per SM walks 128-row tiles of x.  The hidden dimension is cut in
// 8 chunks of 64 units; for each chunk
//   GEMM1  acc1[128 x (64 value | 64 gate)] = x̂_tile · W1chunkᵀ   (tcgen05, K = 128; x̂ = the tile's rows after the
//          LayerNorm, rounded to bf16 as the eager module's LayerNorm output is, A operand in tensor memory)
//   SwiGLU one thread per row: TMEM -> registers, silu via tanh (gate rows of W1 are packed halved), product -> bf16
//          tile H in tensor memory (A operand of the next GEMM)
//   GEMM2  acc2[128 x 128] += H · W2chunkᵀ                        (tcgen05, K = 64)
// W1/W2 chunks stream from L2 through two TMA rings; GEMM1 of chunk j+1 is issued before
// GEMM2 of chunk j so the tensor core runs while the SwiGLU warps work.
//
// Warp roles (512 threads): warps 0-3 / 4-7 SwiGLU + output warpgroups (even / odd chunks), warp 8 TMA producer of
// x (residual copy) and W1, warp 11 TMA producer of W2, warp 9 GEMM1 issuer / TMEM owner, warp 10 GEMM2 issuer (both
// warp-collective), warps 12-15 row preparation: they load the next tile's rows a second time into a staging tile,
// layer-normalise them in place while the current tile's GEMMs run and copy them to tensor memory at the tile switch.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kThreads = 512;
constexpr int kTileM = 128;
constexpr int kChunk = 64;                 // hidden units per chunk
constexpr int kChunks = kHidden / kChunk;  // 8

struct TransParams {
  long long rows;
  int num_tiles;
  const float2* sc;  // [1024] {unused, bias} of the W1 rows (ReLU form)
  const float* ln;   // gamma[128] | beta[128]
  const int* flags;  // flags[0] != 0 -> apply LayerNorm statistics
  const float* b2;   // [128] bias of the second linear (ReLU form)
  const __nv_bfloat16* mask;
  float eps;
  int add_residual;
  int* status;
  // scatter form (num_peers > 0): the input is a column shard [B][tokens][cols][128]; row (b, i, j) is stored to
  // GPU i / cols at row (b, i % cols, col0 + j) of its row shard [B][cols][tokens][128]
  int num_peers;
  int cols;
  int tokens;
  int col0;
};

constexpr int kMaxPeers = 8;
// One output map per GPU; the plain form uses m[0] only.
struct OutMaps {
  CUtensorMap m[kMaxPeers];
};

// shared memory map
constexpr int kSmX = 0;                        // 2 x 32 KiB
constexpr int kSmW1 = kSmX + 2 * 32768;        // 2 x 32 KiB: [k-half][64 value rows | 64 gate rows][64 ch]
constexpr int kSmW2 = kSmW1 + 2 * 32768;       // 2 x 16 KiB: [128 out rows][64 hidden]
constexpr int kSmXn = kSmW2 + 2 * 16384;       // 2 x 16 KiB: the next tile's normalised rows, [channel half][128 rows][64 ch]
constexpr int kSmOut = kSmXn + 2 * 16384;      // 8 warps x 2 KiB staging slabs
constexpr int kSmSc = kSmOut + 8 * 2048;       // per pair of hidden units {rowsum0, rowsum1, const0, const1}: 256 value pairs, 256 gate pairs
constexpr int kSmLn = kSmSc + 2 * 4096;        // gamma[128] | beta[128] as floats
constexpr int kSmBars = kSmLn + 1024;
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

enum Bar {
  X_FULL = 0, X_EMPTY = 2, W1_FULL = 4, W1_EMPTY = 6, W2_FULL = 8, W2_EMPTY = 10,
  ACC1_FULL = 12, ACC1_FREE = 14, H_FULL = 16, H_FREE = 18, ACC2_FULL = 20, ACC2_FREE = 21, XH_FULL = 22, XH_FREE = 23,
  XN_FULL = 24, XN_EMPTY = 25, NUM_BARS = 26
};

// Tensor memory: two GEMM1 accumulators (64 value + 64 gate columns each), the tile's output accumulator, the
// tile's rows as the A operand of GEMM1 (128 bf16 channels = 64 columns) and two H buffers (64 bf16 hidden units
// = 32 columns each) as the A operand of GEMM2.  Both A operands live here and not in shared memory because a
// tcgen05.mma reads its shared-memory operands again for every instruction: with x and H in shared memory the
// kernel moved ~216 KB through shared memory per chunk (1700 clocks at 128 B/clk) against 768 clocks of tensor
// work.
constexpr uint32_t kTmemAcc1 = 0, kTmemAcc2 = 256, kTmemX = 384, kTmemH = 448, kTmemCols = 512;

// Row m of an x tile in shared memory ([2 channel halves][128 rows][64 ch], 128-byte swizzle) -> the same row,
// layer-normalised and rounded to bf16 as the eager module's LayerNorm output is, in the staging tile (same
// layout).  Two streaming passes over the row (shifted sums, normalise) in packed fp32x2 math with four
// independent accumulators each, so that the thread needs few registers.  `ln` = {gamma[128], beta[128]} in shared
// memory; normalize == false copies the raw row.
__device__ __forceinline__ void prepare_row(uint32_t x0, int m, bool normalize, float eps, const float* ln,
                                            uint32_t stage0) {
  float rstd = 1.f, nmr = 0.f;
  if (normalize) {
    // One pass: sums of (x - k) and (x - k)^2 with k = the row's first channel (a shift keeps the variance
    // formula E[d^2] - E[d]^2 free of cancellation when the row has a large common offset).
    const float k = bf16_lo(lds128(x0 + sw128_offset(m, 0)).x);
    const uint64_t nk2 = pack_f32x2(-k, -k);
    uint64_t sa[4] = {0ull, 0ull, 0ull, 0ull}, sq[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll 8
    for (int c = 0; c < 16; ++c) {
      const uint4 x = lds128(x0 + (c >> 3) * 16384 + sw128_offset(m, c & 7));
      const uint64_t d0 = add_f32x2(pack_f32x2(bf16_lo(x.x), bf16_hi(x.x)), nk2);
      const uint64_t d1 = add_f32x2(pack_f32x2(bf16_lo(x.y), bf16_hi(x.y)), nk2);
      const uint64_t d2 = add_f32x2(pack_f32x2(bf16_lo(x.z), bf16_hi(x.z)), nk2);
      const uint64_t d3 = add_f32x2(pack_f32x2(bf16_lo(x.w), bf16_hi(x.w)), nk2);
      sa[0] = add_f32x2(sa[0], d0), sa[1] = add_f32x2(sa[1], d1), sa[2] = add_f32x2(sa[2], d2), sa[3] = add_f32x2(sa[3], d3);
      sq[0] = fma_f32x2(d0, d0, sq[0]), sq[1] = fma_f32x2(d1, d1, sq[1]);
      sq[2] = fma_f32x2(d2, d2, sq[2]), sq[3] = fma_f32x2(d3, d3, sq[3]);
    }
    float a0, a1, q0, q1;
    unpack_f32x2(add_f32x2(add_f32x2(sa[0], sa[1]), add_f32x2(sa[2], sa[3])), a0, a1);
    unpack_f32x2(add_f32x2(add_f32x2(sq[0], sq[1]), add_f32x2(sq[2], sq[3])), q0, q1);
    const float md = (a0 + a1) * (1.f / kC);  // mean of x - k
    const float var = fmaxf((q0 + q1) * (1.f / kC) - md * md, 0.f);
    rstd = rsqrtf(var + eps);
    nmr = -(md + k) * rstd;
  }
  const uint64_t rstd2 = pack_f32x2(rstd, rstd), nmr2 = pack_f32x2(nmr, nmr);
#pragma unroll 4
  for (int c = 0; c < 16; ++c) {
    const uint32_t off = (c >> 3) * 16384 + sw128_offset(m, c & 7);
    uint4 x = lds128(x0 + off);
    if (normalize) {
      // gamma * (x - mu) * rstd + beta = x * (rstd * gamma) + (beta - mu * rstd * gamma); 8 channels per step
      const float4 g0 = reinterpret_cast<const float4*>(ln)[2 * c], g1 = reinterpret_cast<const float4*>(ln)[2 * c + 1];
      const float4 b0 = reinterpret_cast<const float4*>(ln + kC)[2 * c], b1 = reinterpret_cast<const float4*>(ln + kC)[2 * c + 1];
      auto norm2 = [&](uint32_t w, float ga, float gb, float ba, float bb) -> uint32_t {
        const uint64_t g2 = pack_f32x2(ga, gb);
        const uint64_t y2 = fma_f32x2(pack_f32x2(bf16_lo(w), bf16_hi(w)), mul_f32x2(rstd2, g2),
                                      fma_f32x2(nmr2, g2, pack_f32x2(ba, bb)));
        float y0, y1;
        unpack_f32x2(y2, y0, y1);
        return pack_bf16x2(y0, y1);
      };
      x.x = norm2(x.x, g0.x, g0.y, b0.x, b0.y);
      x.y = norm2(x.y, g0.z, g0.w, b0.z, b0.w);
      x.z = norm2(x.z, g1.x, g1.y, b1.x, b1.y);
      x.w = norm2(x.w, g1.z, g1.w, b1.z, b1.w);
    }
    sts128(stage0 + off, x);
  }
}

// This thread's staged row (both channel halves) -> its lane of the A operand of GEMM1 in tensor memory.
__device__ __forceinline__ void staged_row_to_tmem(uint32_t stage0, int m, uint32_t taddr) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t h[32];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 x = lds128(stage0 + half * 16384 + sw128_offset(m, c));
      h[c * 4 + 0] = x.x, h[c * 4 + 1] = x.y, h[c * 4 + 2] = x.z, h[c * 4 + 3] = x.w;
    }
    tmem_st32(taddr + half * 32, h);
  }
  tmem_st_wait();
}

template <bool kRelu>
__global__ void __launch_bounds__(kThreads, 1)
transition_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w1,
                  const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ OutMaps tm_outs,
                  const TransParams p) {
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + (X_FULL + i) * 8, 1);
      mbar_init(bars + (X_EMPTY + i) * 8, 8);  // the 8 epilogue warps (residual)
      mbar_init(bars + (W1_FULL + i) * 8, 1);
      mbar_init(bars + (W1_EMPTY + i) * 8, 1);
      mbar_init(bars + (W2_FULL + i) * 8, 1);
      mbar_init(bars + (W2_EMPTY + i) * 8, 1);
      mbar_init(bars + (ACC1_FULL + i) * 8, 1);
      mbar_init(bars + (ACC1_FREE + i) * 8, 4);
      mbar_init(bars + (H_FULL + i) * 8, 4);
      mbar_init(bars + (H_FREE + i) * 8, 1);
    }
    mbar_init(bars + ACC2_FULL * 8, 1);
    mbar_init(bars + ACC2_FREE * 8, 8);
    mbar_init(bars + XH_FULL * 8, 4);
    mbar_init(bars + XH_FREE * 8, 1);
    mbar_init(bars + XN_FULL * 8, 1);
    mbar_init(bars + XN_EMPTY * 8, 4);
    fence_mbar_init();
  }
  // stage the constants: LayerNorm gamma | beta, and for the ReLU form the two linears' biases
  if (threadIdx.x < 2 * kC) reinterpret_cast<float*>(gen + kSmLn)[threadIdx.x] = p.ln[threadIdx.x];
  if (kRelu) {
    for (int q = threadIdx.x; q < kHidden; q += kThreads) reinterpret_cast<float*>(gen + kSmSc)[q] = p.sc[q].y;
    if (threadIdx.x < kC) reinterpret_cast<float*>(gen + kSmSc + 4096)[threadIdx.x] = p.b2[threadIdx.x];
  }
  if (warp == 9) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int my_tiles = (p.num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;

  // Register budget: 128 per thread at launch; the two helper warpgroups hand registers to the two SwiGLU
  // warpgroups, which hold a whole accumulator row (128 values) at a time: 128 x 56 + 128 x 72 + 256 x 192 = 512 x 128.
  if (warp >= 12) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  } else if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  }
  if (warp >= 12) {
    // ------------------------------------------------------------------ row preparation warpgroup
    // Thread = row.  The warpgroup loads the tile's rows a second time, by its own TMA request into the staging
    // tile, as soon as that tile is free (right after the previous copy, i.e. when the GEMMs of the tile before
    // start) — the x ring's slots, which only feed the residual now, free too late for that.  It layer-normalises the
    // rows in place and, once GEMM1 has finished with the previous tile, copies them into tensor memory as the A
    // operand of GEMM1.  Only the copy sits on the tile switch's critical path.
    const int m = (warp & 3) * 32 + lane;
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const bool normalize = __ldg(p.flags) != 0;
    const float* ln_s = reinterpret_cast<const float*>(gen + kSmLn);
    const uint32_t xn = base + kSmXn;
    auto request_rows = [&](int i) {  // one thread; the staging tile is free
      const int tile = blockIdx.x + i * gridDim.x;
      mbar_expect_tx(bars + XN_FULL * 8, 32768);
      tma_load_2d(xn, &tm_x, bars + XN_FULL * 8, 0, tile * kTileM);
      tma_load_2d(xn + 16384, &tm_x, bars + XN_FULL * 8, 64, tile * kTileM);
    };
    int requested = 0;
    if (warp == 12 && lane == 0) request_rows(0), ++requested;
    bool ok = true;
    for (int i = 0; ok && i < my_tiles; ++i) {
      ok = mbar_wait(bars + XN_FULL * 8, i & 1, abort_flag);
      if (!ok) break;
      prepare_row(xn, m, normalize, p.eps, ln_s, xn);
      if (i > 0) {  // GEMM1 has read the previous tile's rows for the last time once its last chunk is complete
        ok = mbar_wait(bars + XH_FREE * 8, (i - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
      }
      staged_row_to_tmem(xn, m, lane_taddr + kTmemX);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + XH_FULL * 8);
      // once all 128 rows have been copied the staging tile can take the next tile's rows
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + XN_EMPTY * 8);
      if (warp == 12 && lane == 0 && i + 1 < my_tiles) {
        ok = mbar_wait(bars + XN_EMPTY * 8, i & 1, abort_flag);
        if (ok) request_rows(i + 1), ++requested;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
    }
    // (on an abandoned wait a request may still be in flight: give it a bounded chance to land)
    if (*abort_flag && warp == 12 && lane == 0 && requested > 0)
      mbar_wait(bars + XN_FULL * 8, (requested - 1) & 1, abort_flag + 1);
  } else
 if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer of x tiles and W1 chunks
    // (what GEMM1 needs; W2 has its own producer so that a W2 slot that frees late never holds back a W1 load)
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w1);
      tma_prefetch_desc(&tm_outs.m[0]);
      bool ok = true;
      int c = 0;  // chunk counter
      auto load_x = [&](int i) -> bool {
        const int xs = i & 1;
        if (!mbar_wait(bars + (X_EMPTY + xs) * 8, ((i >> 1) & 1) ^ 1, abort_flag)) return false;
        mbar_expect_tx(bars + (X_FULL + xs) * 8, 32768);
        const int tile = blockIdx.x + i * gridDim.x;
        tma_load_2d(base + kSmX + xs * 32768, &tm_x, bars + (X_FULL + xs) * 8, 0, tile * kTileM);
        tma_load_2d(base + kSmX + xs * 32768 + 16384, &tm_x, bars + (X_FULL + xs) * 8, 64, tile * kTileM);
        return true;
      };
      ok = load_x(0);
      for (int i = 0; ok && i < my_tiles; ++i) {
        for (int j = 0; j < kChunks; ++j, ++c) {
          const int st = c & 1;
          ok = mbar_wait(bars + (W1_EMPTY + st) * 8, ((c >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t f1 = bars + (W1_FULL + st) * 8;
          mbar_expect_tx(f1, 32768);
          for (int kh = 0; kh < 2; ++kh) {
            const uint32_t dst = base + kSmW1 + st * 32768 + kh * 16384;
            tma_load_2d(dst, &tm_w1, f1, kh * 64, j * kChunk);                  // value rows
            tma_load_2d(dst + 8192, &tm_w1, f1, kh * 64, kHidden + j * kChunk);  // gate rows
          }
          // the next tile's rows, early enough for the SwiGLU warpgroups to normalise them during this tile
          if (j == 2 && i + 1 < my_tiles) {
            ok = load_x(i + 1);
            if (!ok) break;
          }
        }
      }
      if (*abort_flag && c > 0) {
        const int last = c - 1;
        mbar_wait(bars + (W1_FULL + (last & 1)) * 8, (last >> 1) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------ TMA producer of W2 chunks
    if (lane == 0) {
      tma_prefetch_desc(&tm_w2);
      bool ok = true;
      int c = 0;
      for (int i = 0; ok && i < my_tiles; ++i) {
        for (int j = 0; j < kChunks; ++j, ++c) {
          const int st = c & 1;
          ok = mbar_wait(bars + (W2_EMPTY + st) * 8, ((c >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t f2 = bars + (W2_FULL + st) * 8;
          mbar_expect_tx(f2, 16384);
          tma_load_2d(base + kSmW2 + st * 16384, &tm_w2, f2, j * kChunk, 0);
        }
      }
      if (*abort_flag && c > 0) {
        const int last = c - 1;
        mbar_wait(bars + (W2_FULL + (last & 1)) * 8, (last >> 1) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ GEMM1 issuer
    // The whole warp runs the loop with the same values and one elected lane issues (umma_*_warp): a converged
    // warp issues an MMA at the rate the tensor pipe retires it, a single thread in a branch about half as fast.
    {
      const uint32_t idesc = make_idesc_bf16(kTileM, 128);
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      bool ok = true;
      int c1 = 0;  // chunk counter
      for (int i = 0; ok && i < my_tiles; ++i) {
        ok = mbar_wait_warp(bars + XH_FULL * 8, i & 1, abort_flag);  // the tile's rows are in tensor memory
        if (!ok) break;
        for (int j = 0; ok && j < kChunks; ++j, ++c1) {
          const int e = c1 & 1;
          const uint32_t par = (c1 >> 1) & 1;
          ok = mbar_wait_warp(bars + (W1_FULL + e) * 8, par, abort_flag) &&
               mbar_wait_warp(bars + (ACC1_FREE + e) * 8, par ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          // one descriptor per operand; each K step adds a constant to the address field (16-byte units)
          const uint64_t db = make_smem_desc(base + kSmW1 + e * 32768, 16, 1024, kLayoutSw128);
          const uint32_t d1 = tb + kTmemAcc1 + e * 128;
#pragma unroll
          for (int k = 0; k < 8; ++k) {  // 16 channels per step: 8 columns of the A operand
            const uint32_t off = (k >> 2) * (16384 >> 4) + (k & 3) * 2;
            umma_ts_warp(d1, tb + kTmemX + k * 8, db + off, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit_warp(bars + (ACC1_FULL + e) * 8);
          umma_commit_warp(bars + (W1_EMPTY + e) * 8);
          if (j == kChunks - 1) umma_commit_warp(bars + XH_FREE * 8);  // the next tile's rows may replace this tile's
        }
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ GEMM2 issuer (warp-collective as well)
    {
      const uint32_t idesc = make_idesc_bf16(kTileM, 128);
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      bool ok = true;
      int c2 = 0;  // chunk counter
      for (int i = 0; ok && i < my_tiles; ++i) {
        for (int jj = 0; ok && jj < kChunks; ++jj, ++c2) {
          const int e = c2 & 1;
          const uint32_t par = (c2 >> 1) & 1;
          ok = mbar_wait_warp(bars + (W2_FULL + e) * 8, par, abort_flag) &&
               mbar_wait_warp(bars + (H_FULL + e) * 8, par, abort_flag);
          if (ok && jj == 0) ok = mbar_wait_warp(bars + ACC2_FREE * 8, (i & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dw = make_smem_desc(base + kSmW2 + e * 16384, 16, 1024, kLayoutSw128);
          const uint32_t d2 = tb + kTmemAcc2, th = tb + kTmemH + e * 32;
          umma_ts_warp(d2, th, dw, idesc, jj > 0 ? 1u : 0u);
#pragma unroll
          for (int k = 1; k < 4; ++k) umma_ts_warp(d2, th + k * 8, dw + k * 2, idesc, 1u);
          umma_commit_warp(bars + (W2_EMPTY + e) * 8);
          umma_commit_warp(bars + (H_FREE + e) * 8);
          if (jj == kChunks - 1) umma_commit_warp(bars + ACC2_FULL * 8);
        }
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ SwiGLU / output warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 192;");
    const int e = warp >> 2;               // chunk parity and output column half this warpgroup owns
    const int m = (warp & 3) * 32 + lane;  // row inside the tile == TMEM lane
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t slab = base + kSmOut + warp * 2048;
    bool ok = true;
    int n = 0;  // uses of this warpgroup's acc1 / H buffers
    for (int i = 0; ok && i < my_tiles; ++i) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int xs = i & 1;
      const long long row = (long long)tile * kTileM + m;
      const uint32_t x0 = base + kSmX + xs * 32768;
      for (int j = e; ok && j < kChunks; j += 2, ++n) {
        ok = mbar_wait(bars + (ACC1_FULL + e) * 8, n & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        // The whole accumulator (64 value and 64 gate columns of this row) goes to registers first, so that it is
        // free for the chunk after next while this one is still being computed.
        uint32_t xv[64], xg[64];
        const uint32_t acc1 = lane_taddr + kTmemAcc1 + e * 128;
        tmem_ld32(acc1, reinterpret_cast<uint32_t(&)[32]>(xv[0]));
        tmem_ld32(acc1 + 32, reinterpret_cast<uint32_t(&)[32]>(xv[32]));
        if (!kRelu) {
          tmem_ld32(acc1 + 64, reinterpret_cast<uint32_t(&)[32]>(xg[0]));
          tmem_ld32(acc1 + 96, reinterpret_cast<uint32_t(&)[32]>(xg[32]));
        }
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (ACC1_FREE + e) * 8);
        // the H buffer's previous use (two chunks back) must have been consumed by its GEMM2 (long done as a rule)
        ok = mbar_wait(bars + (H_FREE + e) * 8, (n & 1) ^ 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int half = 0; half < 2; ++half) {  // 32 hidden units at a time -> 16 columns of the A operand of GEMM2
          uint32_t pk[16];
          if (kRelu) {
            const float2* b1s = reinterpret_cast<const float2*>(gen + kSmSc) + j * (kChunk / 2) + half * 16;
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              const float2 b = b1s[t];
              const int u = half * 32 + 2 * t;
              pk[t] = pack_bf16x2(fmaxf(__uint_as_float(xv[u]) + b.x, 0.f), fmaxf(__uint_as_float(xv[u + 1]) + b.y, 0.f));
            }
          } else {
#pragma unroll
            for (int t = 0; t < 16; ++t) {
              // two hidden units at a time, packed fp32x2 math; the gate rows of W1 are halved when they are
              // packed: silu(gate) * value = (h * tanh(h) + h) * value with h = gate / 2
              const int u = half * 32 + 2 * t;
              const float h0 = __uint_as_float(xg[u]), h1 = __uint_as_float(xg[u + 1]);
              const uint64_t h2 = pack_f32x2(h0, h1);
              const uint64_t hid2 = mul_f32x2(fma_f32x2(h2, pack_f32x2(tanh_approx(h0), tanh_approx(h1)), h2),
                                              pack_f32x2(__uint_as_float(xv[u]), __uint_as_float(xv[u + 1])));
              float o0, o1;
              unpack_f32x2(hid2, o0, o1);
              pk[t] = pack_bf16x2(o0, o1);
            }
          }
          tmem_st16(lane_taddr + kTmemH + e * 32 + half * 16, pk);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (H_FULL + e) * 8);
      }
      if (!ok) break;
      // ---- output: columns [64e, 64e+64) of acc2 (+ residual) (* mask)
      ok = mbar_wait(bars + ACC2_FULL * 8, i & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t acc[64];
      tmem_ld32(lane_taddr + kTmemAcc2 + e * 64, reinterpret_cast<uint32_t(&)[32]>(acc[0]));
      tmem_ld32(lane_taddr + kTmemAcc2 + e * 64 + 32, reinterpret_cast<uint32_t(&)[32]>(acc[32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + ACC2_FREE * 8);  // the next tile's GEMM2 may start
      if (p.add_residual) {  // (long complete: the wait only orders this thread's reads after the TMA writes)
        ok = mbar_wait(bars + (X_FULL + xs) * 8, (i >> 1) & 1, abort_flag);
        if (!ok) break;
      }
      float mk = 1.f;
      if (p.mask != nullptr && row < p.rows) mk = __bfloat162float(p.mask[row]);
#pragma unroll
      for (int g = 0; g < 2; ++g) {
        const uint32_t* a = acc + g * 32;
        uint32_t res[16];
        if (p.add_residual) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 x = lds128(x0 + e * 16384 + sw128_offset(m, g * 4 + c));
            res[c * 4 + 0] = x.x, res[c * 4 + 1] = x.y, res[c * 4 + 2] = x.z, res[c * 4 + 3] = x.w;
          }
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t) res[t] = 0u;
        }
        uint32_t pk[16];
        if (kRelu) {
          const float* b2s = reinterpret_cast<const float*>(gen + kSmSc + 4096) + e * 64 + g * 32;
#pragma unroll
          for (int t = 0; t < 16; ++t)
            pk[t] = pack_bf16x2(fmaf(mk, __uint_as_float(a[2 * t]) + b2s[2 * t], bf16_lo(res[t])),
                                fmaf(mk, __uint_as_float(a[2 * t + 1]) + b2s[2 * t + 1], bf16_hi(res[t])));
        } else {
#pragma unroll
          for (int t = 0; t < 16; ++t)
            pk[t] = pack_bf16x2(fmaf(mk, __uint_as_float(a[2 * t]), bf16_lo(res[t])),
                                fmaf(mk, __uint_as_float(a[2 * t + 1]), bf16_hi(res[t])));
        }
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; ++c)
          sts128(slab + sw64_offset(lane, c), make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const long long row0 = (long long)tile * kTileM + (warp & 3) * 32;
          const CUtensorMap* tm = &tm_outs.m[0];
          long long dst0 = row0;
          if (p.num_peers > 0) {  // 32 consecutive rows share (b, i): cols is a multiple of 32
            const long long bi = row0 / p.cols;
            const int j = int(row0 - bi * p.cols), i = int(bi % p.tokens), b = int(bi / p.tokens);
            const int peer = i / p.cols;
            tm = &tm_outs.m[peer];
            dst0 = ((long long)b * p.cols + (i - peer * p.cols)) * p.tokens + p.col0 + j;
          }
          if (row0 < p.rows) tma_store_2d(tm, slab, e * 64 + g * 32, int(dst0));
          tma_store_commit();
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bars + (X_EMPTY + xs) * 8);
    }
    if (lane == 0) tma_store_wait_all();
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

}  // namespace
}  // namespace b200ta

namespace b200ta {
namespace {

// outs[0..num_outs): the output (plain form, one entry, row stride os) or every GPU's row shard (scatter form).
int launch_transition(const void* x, int64_t xs, const void* mask, const void* packed, float eps, void* const* outs,
                      int num_outs, int64_t os, int64_t rows, int add_residual, int num_peers, int cols, int tokens,
                      int col0, void* stream, bool relu = false) {
  B200TA_REQUIRE(x && packed && outs, "transition: NULL pointer");
  B200TA_REQUIRE(rows > 0 && rows < (int64_t(1) << 31), "transition: rows=%lld out of range", (long long)rows);
  B200TA_REQUIRE(xs >= kC && xs % 8 == 0 && os >= kC && os % 8 == 0, "transition: row strides must be >= 128 and multiples of 8 elements");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "transition: packed must be 256-byte aligned");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;
  const char* pk = static_cast<const char*>(packed);

  CUtensorMap tm_x, tm_w1, tm_w2;
  OutMaps tm_outs;
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(rows)};
    uint64_t strides[1] = {uint64_t(xs) * 2};
    uint32_t box[2] = {64, 128};
    rc = encode_tensor_map(&tm_x, x, 2, 2, dims, strides, box, SWZ_128, "transition x");
    if (rc != B200TA_OK) return rc;
    uint64_t ostrides[1] = {uint64_t(os) * 2};
    uint32_t obox[2] = {32, 32};
    for (int k = 0; k < kMaxPeers; ++k) {
      const int src = k < num_outs ? k : 0;
      B200TA_REQUIRE(outs[src], "transition: NULL output pointer");
      rc = encode_tensor_map(&tm_outs.m[k], outs[src], 2, 2, dims, ostrides, obox, SWZ_64, "transition out");
      if (rc != B200TA_OK) return rc;
    }
  }
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(kTransRows)};
    uint64_t strides[1] = {uint64_t(kC) * 2};
    uint32_t box[2] = {64, 64};
    rc = encode_tensor_map(&tm_w1, pk + kTransW1Off, 2, 2, dims, strides, box, SWZ_128, "transition w1");
    if (rc != B200TA_OK) return rc;
  }
  {
    uint64_t dims[2] = {uint64_t(kHidden), uint64_t(kC)};
    uint64_t strides[1] = {uint64_t(kHidden) * 2};
    uint32_t box[2] = {64, 128};
    rc = encode_tensor_map(&tm_w2, pk + kTransW2Off, 2, 2, dims, strides, box, SWZ_128, "transition w2");
    if (rc != B200TA_OK) return rc;
  }

  TransParams p{};
  p.rows = rows;
  p.num_tiles = int((rows + kTileM - 1) / kTileM);
  p.sc = reinterpret_cast<const float2*>(pk + kTransScOff);
  p.flags = reinterpret_cast<const int*>(pk + kTransFlagsOff);
  p.b2 = reinterpret_cast<const float*>(pk + kTransB2Off);
  p.ln = reinterpret_cast<const float*>(pk + kTransLnOff);
  p.mask = static_cast<const __nv_bfloat16*>(mask);
  p.eps = eps;
  p.add_residual = add_residual ? 1 : 0;
  p.status = st->status_dev;
  p.num_peers = num_peers, p.cols = cols, p.tokens = tokens, p.col0 = col0;

  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  if (relu) {
    B200TA_CHECK_CUDA(cudaFuncSetAttribute(transition_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
    transition_kernel<true><<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_x, tm_w1, tm_w2, tm_outs, p);
  } else {
    B200TA_CHECK_CUDA(cudaFuncSetAttribute(transition_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
    transition_kernel<false><<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_x, tm_w1, tm_w2, tm_outs, p);
  }
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_transition(const void* x, int64_t xs, const void* mask, const void* packed, float eps, void* out,
                      int64_t os, int64_t rows, int add_residual, void* stream) {
  return b200ta::launch_transition(x, xs, mask, packed, eps, &out, 1, os, rows, add_residual, 0, 0, 0, 0, stream);
}

int b200ta_transition_relu(const void* x, int64_t xs, const void* mask, const void* packed, float eps, void* out,
                           int64_t os, int64_t rows, int add_residual, void* stream) {
  return b200ta::launch_transition(x, xs, mask, packed, eps, &out, 1, os, rows, add_residual, 0, 0, 0, 0, stream, true);
}

int b200ta_transition_scatter(const void* x, const void* mask, const void* packed, float eps, void* const* peer_out,
                              int num_peers, int rank, int B, int tokens, int cols, int add_residual, void* stream) {
  B200TA_REQUIRE(peer_out && num_peers >= 1 && num_peers <= b200ta::kMaxPeers && rank >= 0 && rank < num_peers,
                 "transition_scatter: need 1..%d peers and a rank among them", b200ta::kMaxPeers);
  B200TA_REQUIRE(B > 0 && cols > 0 && cols % 32 == 0 && tokens == cols * num_peers,
                 "transition_scatter: tokens=%d must be cols=%d x peers=%d and cols a multiple of 32", tokens, cols, num_peers);
  return b200ta::launch_transition(x, b200ta::kC, mask, packed, eps, peer_out, num_peers, b200ta::kC,
                                   int64_t(B) * tokens * cols, add_residual, num_peers, cols, tokens, rank * cols, stream);
}

}  // extern "C"
