// Triangle attention core for sm_100a: flash-style, head_dim 32, bf16 in, fp32 softmax.
//
// For every pair row (b, r), head h and query s:
//   o[s,:] = softmax_t( scale * q[s]·k[t] + bias[b,h,s,t] ; t < len[b,r] ) · v[t,:]   (* sigmoid(gate[s,:]))
// The N x N x N logits never exist in memory: a CTA owns 256 queries of one (b, r, h),
// walks the keys in tiles of 128 and keeps running max / sum / output per query.
//
// Per key tile:
//   TMA      K tile, V tile and the two 128x128 bias tiles (one per 128-query half) -> shared memory
//   tcgen05  S = Q·Kᵀ        (128x128x32, both operands K-major in smem, accumulator in TMEM)
//   softmax  one thread per query row: TMEM -> registers, logit = S*scale*log2e + bias (bias is
//            stored pre-multiplied by log2e), running max, exp2, row sum; the bf16 probabilities
//            overwrite the bias tile in place (same swizzled layout = the A operand of the next MMA)
//   tcgen05  O_tile = P·V    (128x32x128, V is the MN-major B operand straight from its [key][d] tile)
//   softmax  accumulates O_tile into registers with the usual rescale.
// The two 128-query halves are handled by two softmax warpgroups that share K/V and
// alternate on the tensor core, so one half's exponentials overlap the other's MMAs.
//
// Warp roles (384 threads): warps 0-3 softmax half 0, warps 4-7 softmax half 1,
// warp 8 TMA producer, warp 9 MMA issuer / TMEM owner, warps 10-11 idle.  The third
// warpgroup gives most of its registers to the softmax warpgroups (setmaxnreg).
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kThreads = 384;  // 3 warpgroups; the third holds the producer and MMA warps
constexpr int kQTile = 128;   // queries per softmax warpgroup
constexpr int kKTile = 128;   // keys per tile
constexpr int kStages = 2;

struct AttnParams {
  int B, R, S, S_pad;
  int q_pairs;    // ceil(S / 256)
  int num_items;  // B * 4 * q_pairs * R
  const int32_t* lengths;
  long long ls_b, ls_r;
  const __nv_bfloat16* gate;
  long long g_br, g_h, g_s;
  __nv_bfloat16* out;
  long long o_br, o_s, o_h;
  float* lse;
  float scale_log2;  // softmax_scale * log2(e)
  int empty_uniform;
  int* status;
};

// shared-memory map (bytes, relative to the 1024-aligned base)
constexpr int kSmQ = 0;                          // 2 item buffers x 2 halves x 8 KiB
constexpr int kSmStage = kSmQ + 2 * 2 * 8192;    // per stage: K 8 KiB, V 8 KiB, bias/P half0 32 KiB, half1 32 KiB
constexpr int kStageBytes = 8192 + 8192 + 2 * 32768;
constexpr int kSmBars = kSmStage + kStages * kStageBytes;
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

enum Bar {
  Q_FULL = 0,    // [2] item buffer
  Q_EMPTY = 2,   // [2]
  KV_FULL = 4,   // [kStages]
  KV_EMPTY = 6,  // [kStages]
  S_FULL = 8,    // [2] per half
  S_FREE = 10,   // [2]
  P_FULL = 12,   // [2]
  O_FULL = 14,   // [2]
  NUM_BARS = 16
};

// TMEM columns: S of half w at w*128, PV tile of half w at 256 + w*32
constexpr uint32_t kTmemS = 0, kTmemO = 256, kTmemCols = 512;

struct Item {
  int b, r, h, q0, br;
  int len;      // keys that take part (S for a uniform row)
  int nkt;      // key tiles
  bool uniform; // no valid key and "uniform" semantics: every logit equal
  bool skip;    // no valid key and "zeros" semantics: nothing to compute
};

__device__ __forceinline__ Item decode_item(const AttnParams& p, int item) {
  Item it;
  it.r = item % p.R;
  int t = item / p.R;
  const int qp = t % p.q_pairs;
  t /= p.q_pairs;
  it.h = t % kHeads;
  it.b = t / kHeads;
  it.q0 = qp * 2 * kQTile;
  it.br = it.b * p.R + it.r;
  int len = p.lengths ? p.lengths[it.b * p.ls_b + it.r * p.ls_r] : p.S;
  len = len < 0 ? 0 : (len > p.S ? p.S : len);
  it.uniform = len == 0 && p.empty_uniform;
  it.skip = len == 0 && !p.empty_uniform;
  it.len = it.uniform ? p.S : len;
  it.nkt = (it.len + kKTile - 1) / kKTile;
  return it;
}

__global__ void __launch_bounds__(kThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                 const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_bias,
                 const AttnParams p) {
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
      mbar_init(bars + (Q_FULL + i) * 8, 1);
      mbar_init(bars + (Q_EMPTY + i) * 8, 1);
      mbar_init(bars + (KV_FULL + i) * 8, 1);
      mbar_init(bars + (KV_EMPTY + i) * 8, 1);
      mbar_init(bars + (S_FULL + i) * 8, 1);
      mbar_init(bars + (S_FREE + i) * 8, 4);
      mbar_init(bars + (P_FULL + i) * 8, 4);
      mbar_init(bars + (O_FULL + i) * 8, 1);
    }
    fence_mbar_init();
  }
  if (warp == 9) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int my_items = (p.num_items - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;

  // Register budget: the third warpgroup keeps 56 registers per thread and the two
  // softmax warpgroups take 224 (128 x 56 + 256 x 224 = the whole register file).
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  }
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_bias);
      int g = 0;   // key tiles issued so far (ring position)
      int qi = 0;  // items that loaded Q so far
      bool ok = true;
      for (int i = 0; ok && i < my_items; ++i) {
        const Item it = decode_item(p, blockIdx.x + i * gridDim.x);
        if (it.skip) continue;
        const int nvalid = (it.q0 + kQTile < p.S) ? 2 : 1;
        const int ib = qi & 1;
        ok = mbar_wait(bars + (Q_EMPTY + ib) * 8, ((qi >> 1) & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bars + (Q_FULL + ib) * 8, nvalid * 8192);
        for (int w = 0; w < nvalid; ++w)
          tma_load_4d(base + kSmQ + (ib * 2 + w) * 8192, &tm_q, bars + (Q_FULL + ib) * 8, 0, it.q0 + w * kQTile,
                      it.h, it.br);
        ++qi;
        for (int kt = 0; kt < it.nkt; ++kt, ++g) {
          const int stage = g % kStages;
          ok = mbar_wait(bars + (KV_EMPTY + stage) * 8, ((g / kStages) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t full = bars + (KV_FULL + stage) * 8;
          const uint32_t sbase = base + kSmStage + stage * kStageBytes;
          mbar_expect_tx(full, 16384 + (it.uniform ? 0 : nvalid * 32768));
          tma_load_4d(sbase, &tm_k, full, 0, kt * kKTile, it.h, it.br);
          tma_load_4d(sbase + 8192, &tm_v, full, 0, kt * kKTile, it.h, it.br);
          if (!it.uniform)
            for (int w = 0; w < nvalid; ++w)
              for (int half = 0; half < 2; ++half)
                tma_load_4d(sbase + 16384 + w * 32768 + half * 16384, &tm_bias, full, kt * kKTile + half * 64,
                            it.q0 + w * kQTile, it.h, it.b);
        }
      }
      if (*abort_flag && g > 0) {
        const int last = g - 1;
        mbar_wait(bars + (KV_FULL + last % kStages) * 8, (last / kStages) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(kQTile, kKTile);
      const uint32_t idesc_o = make_idesc_bf16(kQTile, kHeadDim, false, true);
      int g = 0, qi = 0;
      int cs[2] = {0, 0};  // S tiles issued per half
      int cp[2] = {0, 0};  // P tiles consumed per half
      bool ok = true;
      auto issue_s = [&](int w, int ib, int stage) -> bool {
        // S buffer of half w must have been read out by its warpgroup
        if (!mbar_wait(bars + (S_FREE + w) * 8, (cs[w] & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t qa = base + kSmQ + (ib * 2 + w) * 8192;
        const uint32_t ka = base + kSmStage + stage * kStageBytes;
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
          umma_ss(tmem_base + kTmemS + w * 128, make_smem_desc(qa + ks * 32, 16, 512, kLayoutSw64),
                  make_smem_desc(ka + ks * 32, 16, 512, kLayoutSw64), idesc_s, ks > 0 ? 1u : 0u);
        umma_commit(bars + (S_FULL + w) * 8);
        ++cs[w];
        return true;
      };
      for (int i = 0; ok && i < my_items; ++i) {
        const Item it = decode_item(p, blockIdx.x + i * gridDim.x);
        if (it.skip) continue;
        const int nvalid = (it.q0 + kQTile < p.S) ? 2 : 1;
        const int ib = qi & 1;
        ok = mbar_wait(bars + (Q_FULL + ib) * 8, (qi >> 1) & 1, abort_flag);
        if (!ok) break;
        ok = mbar_wait(bars + (KV_FULL + g % kStages) * 8, (g / kStages) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int w = 0; ok && w < nvalid; ++w) ok = issue_s(w, ib, g % kStages);
        for (int kt = 0; ok && kt < it.nkt; ++kt, ++g) {
          const int stage = g % kStages;
          const bool more = kt + 1 < it.nkt;
          if (more) {
            // next tile's scores as soon as its K landed and the S buffers were drained
            ok = mbar_wait(bars + (KV_FULL + (g + 1) % kStages) * 8, ((g + 1) / kStages) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            for (int w = 0; ok && w < nvalid; ++w) ok = issue_s(w, ib, (g + 1) % kStages);
            if (!ok) break;
          } else {
            umma_commit(bars + (Q_EMPTY + ib) * 8);  // every S MMA of this item has been issued
          }
          for (int w = 0; w < nvalid; ++w) {
            ok = mbar_wait(bars + (P_FULL + w) * 8, cp[w] & 1, abort_flag);
            if (!ok) break;
            ++cp[w];
            tc_fence_after();
            const uint32_t pa = base + kSmStage + stage * kStageBytes + 16384 + w * 32768;
            const uint32_t va = base + kSmStage + stage * kStageBytes + 8192;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              umma_ss(tmem_base + kTmemO + w * 32,
                      make_smem_desc(pa + (j >> 2) * 16384 + (j & 3) * 32, 16, 1024, kLayoutSw128),
                      make_smem_desc(va + j * 1024, 16, 512, kLayoutSw64), idesc_o, (kt > 0 || j > 0) ? 1u : 0u);
            umma_commit(bars + (O_FULL + w) * 8);
          }
          if (!ok) break;
          umma_commit(bars + (KV_EMPTY + stage) * 8);
        }
        ++qi;
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int w = warp >> 2;                 // which 128-query half
    const int m = (warp & 3) * 32 + lane;    // query row inside the half == TMEM lane
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    int g = 0;   // ring position (all tiles of all items, same count as the producer)
    int ct = 0;  // tiles this half has processed (phase of S_FULL / O_FULL)
    bool ok = true;
    for (int i = 0; ok && i < my_items; ++i) {
      const Item it = decode_item(p, blockIdx.x + i * gridDim.x);
      const int q = it.q0 + w * kQTile + m;  // query position
      const bool half_valid = it.q0 + w * kQTile < p.S;
      __nv_bfloat16* out_row = p.out + it.br * p.o_br + (long long)q * p.o_s + it.h * p.o_h;
      if (it.skip) {
        if (q < p.S) {
#pragma unroll
          for (int c = 0; c < 4; ++c) reinterpret_cast<uint4*>(out_row)[c] = make_uint4(0, 0, 0, 0);
          if (p.lse) p.lse[((long long)it.br * p.S + q) * kHeads + it.h] = -INFINITY;
        }
        continue;
      }
      if (!half_valid) {
        g += it.nkt;
        continue;
      }
      float row_max = -INFINITY, row_sum = 0.f;

      for (int kt = 0; kt < it.nkt; ++kt, ++g, ++ct) {
        const int stage = g % kStages;
        const uint32_t btile = base + kSmStage + stage * kStageBytes + 16384 + w * 32768;
        ok = mbar_wait(bars + (KV_FULL + stage) * 8, (g / kStages) & 1, abort_flag);
        if (!ok) break;
        ok = mbar_wait(bars + (S_FULL + w) * 8, ct & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        float s2[128];  // raw scores, turned into scaled+biased logits in place
        const uint32_t s_addr = lane_taddr + kTmemS + w * 128;
        // Quarter by quarter (32 keys): TMEM load, the matching 64 bytes of bias, then the
        // scale+bias FMA; keeps only one quarter of bias words in flight.
#define B200TA_SCORE_QUARTER(QI)                                                                       \
  {                                                                                                    \
    tmem_ld32_f128<QI * 32>(s_addr + QI * 32, s2);                                                     \
    uint4 bv[4];                                                                                       \
    _Pragma("unroll") for (int c = 0; c < 4; ++c) bv[c] =                                              \
        lds128(btile + (QI >> 1) * 16384 + sw128_offset(m, (QI & 1) * 4 + c));                         \
    tmem_ld_wait();                                                                                    \
    _Pragma("unroll") for (int c = 0; c < 4; ++c) {                                                    \
      const uint32_t bw[4] = {bv[c].x, bv[c].y, bv[c].z, bv[c].w};                                     \
      _Pragma("unroll") for (int e = 0; e < 4; ++e) {                                                  \
        const int j0 = QI * 32 + c * 8 + 2 * e;                                                        \
        s2[j0] = fmaf(s2[j0], p.scale_log2, bf16_lo(bw[e]));                                           \
        s2[j0 + 1] = fmaf(s2[j0 + 1], p.scale_log2, bf16_hi(bw[e]));                                   \
      }                                                                                                \
    }                                                                                                  \
  }
        B200TA_SCORE_QUARTER(0)
        B200TA_SCORE_QUARTER(1)
        B200TA_SCORE_QUARTER(2)
        B200TA_SCORE_QUARTER(3)
#undef B200TA_SCORE_QUARTER
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (S_FREE + w) * 8);

        if (it.uniform) {
          // no valid key, eager semantics: every logit is the same (the bias tile was not loaded)
#pragma unroll
          for (int j = 0; j < 128; ++j) s2[j] = 0.f;
        }
        const int rem = it.len - kt * kKTile;  // valid keys in this tile
        if (rem < kKTile) {
#pragma unroll
          for (int j = 0; j < 128; ++j)
            if (j >= rem) s2[j] = -INFINITY;
        }
        float tile_max = -INFINITY;
#pragma unroll
        for (int j = 0; j < 128; ++j) tile_max = fmaxf(tile_max, s2[j]);
        // Lazy running max: the reference point of the exponentials only moves when the
        // true max has grown by more than 2^8, so most tiles need no rescale of O.
        float alpha = 1.f;
        if (kt == 0) {
          row_max = tile_max;
        } else if (tile_max > row_max + 8.f) {
          alpha = ex2_approx(row_max - tile_max);
          row_max = tile_max;
        }
        float tile_sum = 0.f;
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          uint32_t pk[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float p0 = ex2_approx(s2[c * 8 + 2 * e] - row_max);
            const float p1 = ex2_approx(s2[c * 8 + 2 * e + 1] - row_max);
            tile_sum += p0 + p1;
            pk[e] = pack_bf16x2(p0, p1);
          }
          sts128(btile + (c >> 3) * 16384 + sw128_offset(m, c & 7), make_uint4(pk[0], pk[1], pk[2], pk[3]));
        }
        row_sum = fmaf(row_sum, alpha, tile_sum);
        if (kt > 0) {
          // the previous tile's P·V must have landed in O before O is rescaled or added to
          ok = mbar_wait(bars + (O_FULL + w) * 8, (ct - 1) & 1, abort_flag);
          if (!ok) break;
          if (__any_sync(0xffffffffu, alpha != 1.f)) {
            tc_fence_after();
            uint32_t t[32];
            tmem_ld32(lane_taddr + kTmemO + w * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) t[j] = __float_as_uint(__uint_as_float(t[j]) * alpha);
            tmem_st32(lane_taddr + kTmemO + w * 32, t);
            tmem_st_wait();
            tc_fence_before();
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (P_FULL + w) * 8);
      }
      if (!ok) break;
      // the item's output: O (in TMEM) / row_sum
      ok = mbar_wait(bars + (O_FULL + w) * 8, (ct - 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      float o[32];
      {
        uint32_t t[32];
        tmem_ld32(lane_taddr + kTmemO + w * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(t[j]);
      }
      tc_fence_before();
      if (q < p.S) {
        const float inv = 1.f / row_sum;
        uint32_t pk[16];
        if (p.gate != nullptr) {
          const uint4* gp = reinterpret_cast<const uint4*>(p.gate + it.br * p.g_br + it.h * p.g_h + (long long)q * p.g_s);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 gv = __ldg(gp + c);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // sigmoid(x) = 1 / (1 + 2^(-x*log2e))
              const float s0 = rcp_approx(1.f + ex2_approx(-1.4426950408889634f * bf16_lo(gw[e])));
              const float s1 = rcp_approx(1.f + ex2_approx(-1.4426950408889634f * bf16_hi(gw[e])));
              pk[c * 4 + e] = pack_bf16x2(o[c * 8 + 2 * e] * inv * s0, o[c * 8 + 2 * e + 1] * inv * s1);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[j] = pack_bf16x2(o[2 * j] * inv, o[2 * j + 1] * inv);
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          reinterpret_cast<uint4*>(out_row)[c] = make_uint4(pk[c * 4], pk[c * 4 + 1], pk[c * 4 + 2], pk[c * 4 + 3]);
        if (p.lse)
          p.lse[((long long)it.br * p.S + q) * kHeads + it.h] =
              it.uniform ? -INFINITY : 0.6931471805599453f * (row_max + __log2f(row_sum));
      }
    }
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

extern "C" {

int b200ta_attention(const void* q, const void* k, const void* v, const void* gate, int64_t s_br, int64_t s_h,
                     int64_t s_s, const void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q,
                     const int32_t* lengths, int64_t ls_b, int64_t ls_r, void* out, int64_t os_br, int64_t os_s,
                     int64_t os_h, float* lse, float softmax_scale, int empty_row_mode, int B, int R, int S,
                     int S_pad, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(q && k && v && bias && out, "attention: NULL pointer");
  B200TA_REQUIRE(B > 0 && R > 0 && S > 0, "attention: bad sizes B=%d R=%d S=%d", B, R, S);
  B200TA_REQUIRE(S_pad >= S && S_pad % 8 == 0, "attention: S_pad=%d must be a multiple of 8 and >= S=%d", S_pad, S);
  B200TA_REQUIRE(s_br % 8 == 0 && s_h % 8 == 0 && s_s % 8 == 0 && s_s > 0, "attention: q/k/v strides must be multiples of 8 elements");
  B200TA_REQUIRE(bs_b % 8 == 0 && bs_h % 8 == 0 && bs_q % 8 == 0 && bs_q > 0, "attention: bias strides must be multiples of 8 elements");
  B200TA_REQUIRE(os_br % 8 == 0 && os_s % 8 == 0 && os_h % 8 == 0, "attention: out strides must be multiples of 8 elements");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15u) == 0 && (gate == nullptr || (reinterpret_cast<uintptr_t>(gate) & 15u) == 0),
                 "attention: out and gate must be 16-byte aligned");
  B200TA_REQUIRE(empty_row_mode == B200TA_EMPTY_ROW_ZEROS || empty_row_mode == B200TA_EMPTY_ROW_UNIFORM,
                 "attention: unknown empty_row_mode %d", empty_row_mode);
  const int64_t q_pairs = (S + 255) / 256;
  const int64_t items = int64_t(B) * kHeads * q_pairs * R;
  B200TA_REQUIRE(items < (int64_t(1) << 31), "attention: too many work items");
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  CUtensorMap tm_q, tm_k, tm_v, tm_bias;
  {
    uint64_t dims[4] = {uint64_t(kHeadDim), uint64_t(S), uint64_t(kHeads), uint64_t(B) * R};
    uint64_t strides[3] = {uint64_t(s_s) * 2, uint64_t(s_h) * 2, B * R == 1 ? 64u : uint64_t(s_br) * 2};
    uint32_t box[4] = {32, 128, 1, 1};
    rc = encode_tensor_map(&tm_q, q, 2, 4, dims, strides, box, SWZ_64, "attention q");
    if (rc == B200TA_OK) rc = encode_tensor_map(&tm_k, k, 2, 4, dims, strides, box, SWZ_64, "attention k");
    if (rc == B200TA_OK) rc = encode_tensor_map(&tm_v, v, 2, 4, dims, strides, box, SWZ_64, "attention v");
    if (rc != B200TA_OK) return rc;
  }
  {
    uint64_t dims[4] = {uint64_t(S_pad), uint64_t(S), uint64_t(kHeads), uint64_t(B)};
    uint64_t strides[3] = {uint64_t(bs_q) * 2, uint64_t(bs_h) * 2, B == 1 ? 64u : uint64_t(bs_b) * 2};
    uint32_t box[4] = {64, 128, 1, 1};
    rc = encode_tensor_map(&tm_bias, bias, 2, 4, dims, strides, box, SWZ_128, "attention bias");
    if (rc != B200TA_OK) return rc;
  }

  AttnParams p{};
  p.B = B, p.R = R, p.S = S, p.S_pad = S_pad;
  p.q_pairs = int(q_pairs);
  p.num_items = int(items);
  p.lengths = lengths;
  p.ls_b = ls_b, p.ls_r = ls_r;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.g_br = s_br, p.g_h = s_h, p.g_s = s_s;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.o_br = os_br, p.o_s = os_s, p.o_h = os_h;
  p.lse = lse;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.empty_uniform = empty_row_mode == B200TA_EMPTY_ROW_UNIFORM ? 1 : 0;
  p.status = st->status_dev;

  B200TA_CHECK_CUDA(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
  const int grid = p.num_items < st->num_sms ? p.num_items : st->num_sms;
  attention_kernel<<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, tm_bias, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
