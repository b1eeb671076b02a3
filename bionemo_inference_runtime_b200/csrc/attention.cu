// Triangle attention core for sm_100a: flash-style, head_dim 32, bf16 in, fp32 softmax.
//
// For every pair row (b, r), head h and query s:
//   o[s,:] = softmax_t( scale * (q[s]·k[t] + bias[b,h,s,t]) ; t < len[b,r] ) · v[t,:]   (* gate[s,:])
// where `bias` is the triangle bias already divided by `scale` and `gate` holds sigmoid(gate logits) (the
// prologue writes both that way).
// The N x N x N logits never exist in memory: a CTA owns 256 queries of one (b, r, h), walks the
// keys in tiles of 128 and keeps a reference point and a running sum per query and the output in TMEM.
//
// Everything that touches a score matrix element is either a tensor-core or a TMEM operation:
//   TMA      K tile, V tile and the two 128x128 bias tiles (one per 128-query half) -> shared memory
//   tcgen05  S  = Q·Kᵀ          (128x128x32, K-major operands in smem, accumulator in TMEM)
//   tcgen05  S += I·Bias        (128x128x128: the identity, resident in TMEM as the A operand, times the
//                                bias tile as MN-major B operand - the bias add costs no CUDA-core work)
//   softmax  one thread per query row: S from TMEM -> registers, exp2 relative to the maximum of the row's
//            first key tile, row sum; the bf16 probabilities go straight back to TMEM
//   tcgen05  O += P·V           (128x32x128: P is the A operand from TMEM, V the MN-major B operand from
//                                its [key][d] tile); O is only rescaled when a tile's sum would leave the
//                                safe fp32 range
// The two 128-query halves are handled by two softmax warpgroups that share K/V.  Each half has its own
// score-MMA warp, which runs one key tile ahead (also across work items), so the next scores are in TMEM
// before a warpgroup asks for them.
//
// A pair row without a valid key takes a constant path in "uniform" mode (probabilities all 1: the output is the
// mean of V, as the eager reference computes it) and is skipped in "zeros" mode.
//
// Warp roles (384 threads): warps 0-3 softmax half 0, warps 4-7 softmax half 1, warp 8 TMA producer,
// warps 9 and 11 score-MMA issuers of the two halves (warp 9 owns TMEM), warp 10 P·V-MMA issuer.  The third warpgroup gives most
// of its registers to the softmax warpgroups (setmaxnreg).
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kThreads = 384;
constexpr int kQTile = 128;  // queries per softmax warpgroup
constexpr int kKTile = 128;  // keys per tile
constexpr int kStages = 2;
constexpr float kRebaseSum = 1.2676506e30f;  // 2^100: a tile sum at or above this moves the reference point

struct AttnParams {
  int B, R, S, S_pad;
  int q_pairs;    // ceil(S / 256)
  uint32_t r_mul, r_shr, qp_mul, qp_shr;  // division by R and by q_pairs as multiply-high and shift
  int num_items;  // B * 4 * q_pairs * R
  const int32_t* lengths;
  long long ls_b, ls_r;
  const uint32_t* key_mask;  // masked form: bit k of word [b][r][k / 32] = key k takes part (0 at and past the length)
  long long km_b, km_r;      // strides of key_mask in words
  const __nv_bfloat16* gate;
  long long g_br, g_h, g_s;
  __nv_bfloat16* out;
  long long o_br, o_s, o_h;
  float* lse;
  float scale_log2;  // softmax_scale * log2(e)
  int empty_uniform;
  int wide_store;  // out is 32-byte aligned and its strides are multiples of 16 elements
  int* status;
};

// 32-byte store; the address must be 32-byte aligned.
__device__ __forceinline__ void stg256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// shared-memory map (bytes, relative to the 1024-aligned base)
// K and the bias tiles are only read by the score MMAs, which run a tile ahead, so their ring frees early
// and two stages are enough to hide the load latency; V waits for the probabilities and gets a deeper ring.
constexpr int kVStages = 4;
constexpr int kSmQ = 0;                        // 2 item buffers x 2 halves x 8 KiB
constexpr int kSmStage = kSmQ + 2 * 2 * 8192;  // per stage: K 8 KiB, bias half0 32 KiB, bias half1 32 KiB
constexpr int kStageBytes = 8192 + 2 * 32768;
constexpr int kSmV = kSmStage + kStages * kStageBytes;  // kVStages x 8 KiB
constexpr int kSmBars = kSmV + kVStages * 8192;
constexpr int kSmTotal = kSmBars + 256;
constexpr int kSmDynamic = kSmTotal + 1024;

enum Bar {
  Q_FULL = 0,    // [2] item buffer
  Q_EMPTY = 2,   // [2]
  KB_FULL = 4,   // [kStages] K + bias
  KB_EMPTY = 6,  // [kStages]
  S_FULL = 8,    // [2] per half
  S_FREE = 10,   // [2]
  P_FULL = 12,   // [2]
  O_FULL = 14,   // [2]
  V_FULL = 16,   // [kVStages]
  V_EMPTY = 20,  // [kVStages]
  NUM_BARS = 24
};

// TMEM columns: S of half w | O of half w | P (bf16 pairs) of half w | identity (bf16 pairs)
constexpr uint32_t kTmemS = 0, kTmemO = 256, kTmemP = 320, kTmemI = 448, kTmemCols = 512;

struct Item {
  int b, r, h, q0, br;
  int len;       // keys that take part (S for a uniform row)
  int nkt;       // key tiles
  int nvalid;    // 128-query halves that hold at least one query
  bool uniform;  // no valid key and "uniform" semantics: every logit equal
  bool skip;     // no valid key and "zeros" semantics: nothing to compute
};

// n / d for n < 2^31 with the constants of fast_div_constants(); mul == 0 stands for d == 1.
__device__ __forceinline__ int fast_div(int n, uint32_t mul, uint32_t shr) {
  return mul ? int(__umulhi(uint32_t(n), mul) >> shr) : n;
}

// Row length of a work item as stored (not clamped yet).
__device__ __forceinline__ int item_raw_length(const AttnParams& p, int item) {
  if (p.lengths == nullptr) return p.S;
  const int t = fast_div(item, p.qp_mul, p.qp_shr);
  const int t2 = fast_div(t, p.r_mul, p.r_shr);
  const int r = t - t2 * p.R;
  const int b = t2 / kHeads;
  return p.lengths[b * p.ls_b + r * p.ls_r];
}

__device__ __forceinline__ Item decode_item(const AttnParams& p, int item, int len) {
  Item it;
  // Items are ordered (b, h, r, query pair) with the query pair fastest: the CTAs that run at the same time work
  // on the query tiles of neighbouring pair rows, so a row's K and V come from HBM once (and then from L2) while
  // the head's bias, shared by all rows, stays in L2.
  const int t = fast_div(item, p.qp_mul, p.qp_shr);
  const int qp = item - t * p.q_pairs;
  const int t2 = fast_div(t, p.r_mul, p.r_shr);
  it.r = t - t2 * p.R;
  it.h = t2 % kHeads;
  it.b = t2 / kHeads;
  it.q0 = qp * 2 * kQTile;
  it.br = it.b * p.R + it.r;
  len = len < 0 ? 0 : (len > p.S ? p.S : len);
  it.uniform = len == 0 && p.empty_uniform;
  it.skip = len == 0 && !p.empty_uniform;
  it.len = it.uniform ? p.S : len;
  it.nkt = (it.len + kKTile - 1) / kKTile;
  it.nvalid = (it.q0 + kQTile < p.S) ? 2 : 1;
  return it;
}

// Walks the (item, key tile) sequence of one CTA in order, skipping items without work.
struct TileCursor {
  int i;     // index into this CTA's item list
  int kt;    // key tile inside the item
  int g;     // tiles before this one (ring position)
  int qi;    // items with work before this one (Q buffer position)
  Item it;
  bool valid;
};

// kWarp: called by all lanes of a converged warp; the row length read from memory is broadcast from lane 0 so
// that everything derived from it is the same in every lane by construction (warp-uniform code).
template <bool kWarp = false>
__device__ __forceinline__ void cursor_seek(const AttnParams& p, TileCursor& c, int my_items) {
  // positions the cursor on the first item with work at or after c.i
  while (c.i < my_items) {
    int len = item_raw_length(p, blockIdx.x + c.i * gridDim.x);
    if (kWarp) len = __shfl_sync(0xffffffffu, len, 0);
    c.it = decode_item(p, blockIdx.x + c.i * gridDim.x, len);
    if (!c.it.skip) {
      c.valid = true;
      return;
    }
    ++c.i;
  }
  c.valid = false;
}
template <bool kWarp = false>
__device__ __forceinline__ void cursor_init(const AttnParams& p, TileCursor& c, int my_items) {
  c.i = 0, c.kt = 0, c.g = 0, c.qi = 0;
  cursor_seek<kWarp>(p, c, my_items);
}
template <bool kWarp = false>
__device__ __forceinline__ void cursor_next(const AttnParams& p, TileCursor& c, int my_items) {
  ++c.g;
  if (++c.kt < c.it.nkt) return;
  c.kt = 0;
  ++c.qi;
  ++c.i;
  cursor_seek<kWarp>(p, c, my_items);
}

template <bool kMasked>
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
      mbar_init(bars + (Q_EMPTY + i) * 8, 2);   // one arrival per score-MMA warp
      mbar_init(bars + (KB_FULL + i) * 8, 1);
      mbar_init(bars + (KB_EMPTY + i) * 8, 2);  // one arrival per score-MMA warp
      mbar_init(bars + (S_FULL + i) * 8, 1);
      mbar_init(bars + (S_FREE + i) * 8, 4);
      mbar_init(bars + (P_FULL + i) * 8, 4);
      mbar_init(bars + (O_FULL + i) * 8, 1);
    }
    for (int i = 0; i < kVStages; ++i) {
      mbar_init(bars + (V_FULL + i) * 8, 1);
      mbar_init(bars + (V_EMPTY + i) * 8, 1);
    }
    fence_mbar_init();
  }
  if (warp == 9) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // The 128x128 bf16 identity, A operand of the bias MMA: TMEM lane q, column c holds elements (q, 2c) and
  // (q, 2c+1) as a bf16 pair, so lane q has a single 1.0 in column q/2.
  if (warp < 4) {
    const int q = warp * 32 + lane;
    const uint32_t one = (q & 1) ? 0x3F800000u : 0x00003F80u;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t v[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) v[c] = (half * 32 + c == (q >> 1)) ? one : 0u;
      tmem_st32(tmem_base + (uint32_t(warp * 32) << 16) + kTmemI + half * 32, v);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const int my_items = (p.num_items - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;

  // Register budget.  The CTA starts with 168 registers per thread; setmaxnreg only moves registers inside
  // that allocation, and an increase blocks until a decrease has freed enough: the third warpgroup drops
  // to 72 (frees 128 x 96) and the two softmax warpgroups rise to 216 (need 256 x 48, the same number).
  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  }
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_bias);
      TileCursor c;
      cursor_init(p, c, my_items);
      int issued = 0;
      bool ok = true;
      while (ok && c.valid) {
        const Item& it = c.it;
        if (c.kt == 0) {
          const int ib = c.qi & 1;
          ok = mbar_wait(bars + (Q_EMPTY + ib) * 8, ((c.qi >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
          mbar_expect_tx(bars + (Q_FULL + ib) * 8, it.nvalid * 8192);
          for (int w = 0; w < it.nvalid; ++w)
            tma_load_4d(base + kSmQ + (ib * 2 + w) * 8192, &tm_q, bars + (Q_FULL + ib) * 8, 0, it.q0 + w * kQTile,
                        it.h, it.br);
        }
        // K + bias of this tile (needed first, by the score MMAs)
        const int stage = c.g % kStages;
        ok = mbar_wait(bars + (KB_EMPTY + stage) * 8, ((c.g / kStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        const uint32_t full = bars + (KB_FULL + stage) * 8;
        const uint32_t sbase = base + kSmStage + stage * kStageBytes;
        mbar_expect_tx(full, 8192 + (it.uniform ? 0 : it.nvalid * 32768));
        tma_load_4d(sbase, &tm_k, full, 0, c.kt * kKTile, it.h, it.br);
        if (!it.uniform)
          for (int w = 0; w < it.nvalid; ++w)
            for (int half = 0; half < 2; ++half)
              tma_load_4d(sbase + 8192 + w * 32768 + half * 16384, &tm_bias, full, c.kt * kKTile + half * 64,
                          it.q0 + w * kQTile, it.h, it.b);
        // V of this tile
        const int vs = c.g % kVStages;
        ok = mbar_wait(bars + (V_EMPTY + vs) * 8, ((c.g / kVStages) & 1) ^ 1, abort_flag);
        if (!ok) break;
        mbar_expect_tx(bars + (V_FULL + vs) * 8, 8192);
        tma_load_4d(base + kSmV + vs * 8192, &tm_v, bars + (V_FULL + vs) * 8, 0, c.kt * kKTile, it.h, it.br);
        ++issued;
        cursor_next(p, c, my_items);
      }
      // If the loop was abandoned, give copies still in flight a bounded chance to land.
      if (*abort_flag && issued > 0) {
        const int last = issued - 1;
        mbar_wait(bars + (V_FULL + last % kVStages) * 8, (last / kVStages) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 9 || warp == 11) {
    // ------------------------------------------------------------------ score MMA issuers (S = Q·Kᵀ + I·Bias)
    // One warp per 128-query half.  All 32 lanes run the loop with the same values and one elected lane issues
    // (umma_*_warp): a converged warp issues its MMAs at the rate the tensor pipe retires them, a single thread
    // inside a branch needs 45-80 clocks per MMA.  Each warp runs one key tile ahead of the softmax (also across
    // work items): the only thing it waits for besides the loads is that its half's S buffer has been read out.
    {
      constexpr uint32_t idesc_s = make_idesc_bf16(kQTile, kKTile);                // Q·Kᵀ: both operands K-major
      constexpr uint32_t idesc_b1 = make_idesc_bf16(kQTile, 128, false, true);     // I·Bias: B MN-major
      const int w = __shfl_sync(0xffffffffu, warp == 9 ? 0 : 1, 0);
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      const uint32_t ti = tb + kTmemI;
      const uint32_t d = tb + kTmemS + w * 128;  // S of this half
      int n = 0;                                 // S tiles issued (phase of S_FREE)
      bool ok = true;
      TileCursor c;
      cursor_init<true>(p, c, my_items);
      while (ok && c.valid) {
        const Item& it = c.it;
        const int ib = c.qi & 1, stage = c.g % kStages;
        if (c.kt == 0) ok = mbar_wait_warp(bars + (Q_FULL + ib) * 8, (c.qi >> 1) & 1, abort_flag);
        ok = ok && mbar_wait_warp(bars + (KB_FULL + stage) * 8, (c.g / kStages) & 1, abort_flag);
        if (!ok) break;
        if (w < it.nvalid) {
          // One descriptor per operand tile; the K steps only add a constant to its address field (in 16-byte
          // units).
          const uint32_t sbase = base + kSmStage + stage * kStageBytes;
          const uint64_t dk = make_smem_desc(sbase, 16, 512, kLayoutSw64);
          const uint64_t dq = make_smem_desc(base + kSmQ + ib * 16384 + w * 8192, 16, 512, kLayoutSw64);
          // Bias tiles: [128 query rows][64 keys] blocks with 128-byte swizzle, 16 KiB apart: keys 0-63 and
          // 64-127 of half 0, then of half 1.  As B[key][query] this is MN-major with 16 query rows (2 KiB)
          // per K step.
          const uint64_t db = make_smem_desc(sbase + 8192 + w * 32768, 16384, 1024, kLayoutSw128);
          ok = mbar_wait_warp(bars + (S_FREE + w) * 8, (n & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          if (!it.uniform) {  // a row without a valid key has equal logits: the softmax warps need no scores
            umma_ss_warp(d, dq, dk, idesc_s, 0u);
            umma_ss_warp(d, dq + 2, dk + 2, idesc_s, 1u);  // second 16 channels: +32 bytes
#pragma unroll
            for (int j = 0; j < 8; ++j) umma_ts_warp(d, ti + j * 8, db + j * 128, idesc_b1, 1u);
          }
          umma_commit_warp(bars + (S_FULL + w) * 8);
          ++n;
          umma_commit_warp(bars + (KB_EMPTY + stage) * 8);  // K and bias are free once both halves' MMAs ran
          if (c.kt == it.nkt - 1) umma_commit_warp(bars + (Q_EMPTY + ib) * 8);  // last use of this item's Q
        } else {
          // this half holds no query of the item: only keep the shared barriers' counts complete
          mbar_arrive_warp(bars + (KB_EMPTY + stage) * 8);
          if (c.kt == it.nkt - 1) mbar_arrive_warp(bars + (Q_EMPTY + ib) * 8);
        }
        cursor_next<true>(p, c, my_items);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ P·V MMA issuer (warp-collective as well)
    {
      constexpr uint32_t idesc_o = make_idesc_bf16(kQTile, kHeadDim, false, true);  // P·V: B is MN-major
      const uint32_t tb = __shfl_sync(0xffffffffu, tmem_base, 0);
      int n0 = 0, n1 = 0;  // P tiles consumed per half
      bool ok = true;
      TileCursor c;
      cursor_init<true>(p, c, my_items);
      while (ok && c.valid) {
        const Item& it = c.it;
        const int vs = c.g % kVStages;
        ok = mbar_wait_warp(bars + (V_FULL + vs) * 8, (c.g / kVStages) & 1, abort_flag);
        const uint64_t dv = make_smem_desc(base + kSmV + vs * 8192, 16, 512, kLayoutSw64);
        const uint32_t acc0 = c.kt > 0 ? 1u : 0u;
        ok = ok && mbar_wait_warp(bars + (P_FULL + 0) * 8, n0 & 1, abort_flag);
        if (!ok) break;
        ++n0;
        tc_fence_after();
        {
          const uint32_t d = tb + kTmemO, tp = tb + kTmemP;
          umma_ts_warp(d, tp, dv, idesc_o, acc0);
#pragma unroll
          for (int j = 1; j < 8; ++j) umma_ts_warp(d, tp + j * 8, dv + j * 64, idesc_o, 1u);  // 16 keys = 1 KiB per step
          umma_commit_warp(bars + (O_FULL + 0) * 8);
        }
        if (it.nvalid == 2) {
          ok = mbar_wait_warp(bars + (P_FULL + 1) * 8, n1 & 1, abort_flag);
          if (!ok) break;
          ++n1;
          tc_fence_after();
          const uint32_t d = tb + kTmemO + 32, tp = tb + kTmemP + 64;
          umma_ts_warp(d, tp, dv, idesc_o, acc0);
#pragma unroll
          for (int j = 1; j < 8; ++j) umma_ts_warp(d, tp + j * 8, dv + j * 64, idesc_o, 1u);
          umma_commit_warp(bars + (O_FULL + 1) * 8);
        }
        umma_commit_warp(bars + (V_EMPTY + vs) * 8);
        cursor_next<true>(p, c, my_items);
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int w = warp >> 2;               // which 128-query half
    const int m = (warp & 3) * 32 + lane;  // query row inside the half == TMEM lane
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const uint32_t s_addr = lane_taddr + kTmemS + w * 128;
    const uint32_t o_addr = lane_taddr + kTmemO + w * 32;
    const uint32_t p_addr = lane_taddr + kTmemP + w * 64;
    const float c = p.scale_log2;                 // raw score -> log2-domain logit
    const uint64_t c2 = pack_f32x2(c, c);
    int ct = 0;  // tiles this half has processed (phase of S_FULL / O_FULL)
    bool ok = true;
    int next_len = item_raw_length(p, blockIdx.x);
    for (int i = 0; ok && i < my_items; ++i) {
      const Item it = decode_item(p, blockIdx.x + i * gridDim.x, next_len);
      // fetch the next item's row length now: its global-memory latency hides behind this item's work
      if (i + 1 < my_items) next_len = item_raw_length(p, blockIdx.x + (i + 1) * gridDim.x);
      const int q = it.q0 + w * kQTile + m;  // query position
      __nv_bfloat16* out_row = p.out + it.br * p.o_br + (long long)q * p.o_s + it.h * p.o_h;
      if (it.skip) {
        if (q < p.S) {
#pragma unroll
          for (int j = 0; j < 4; ++j) reinterpret_cast<uint4*>(out_row)[j] = make_uint4(0, 0, 0, 0);
          if (p.lse) p.lse[((long long)it.br * p.S + q) * kHeads + it.h] = -INFINITY;
        }
        continue;
      }
      if (w >= it.nvalid) continue;  // this half holds no query of the item
      float row_max = 0.f, row_sum = 0.f;  // row_max: reference point of the exponentials, in raw score units
      bool have_anchor = false;            // masked form: a key tile with a valid key has been seen
      uint4 gv[4];                               // gate row, fetched during the last key tile
#pragma unroll
      for (int j = 0; j < 4; ++j) gv[j] = make_uint4(0, 0, 0, 0);

      for (int kt = 0; kt < it.nkt; ++kt, ++ct) {
        if (kt == it.nkt - 1 && p.gate != nullptr && q < p.S) {
          const uint4* gp = reinterpret_cast<const uint4*>(p.gate + it.br * p.g_br + it.h * p.g_h + (long long)q * p.g_s);
#pragma unroll
          for (int j = 0; j < 4; ++j) gv[j] = __ldg(gp + j);
        }
        ok = mbar_wait(bars + (S_FULL + w) * 8, ct & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (it.uniform) {
          // No valid key, eager semantics: every logit is the same, so every probability of the tile is 1 (0 past
          // the last key) and the output becomes the mean of V.  No scores are read, no exponentials taken.
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + (S_FREE + w) * 8);
          if (kt > 0) {
            ok = mbar_wait(bars + (O_FULL + w) * 8, (ct - 1) & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
          }
          const int rem = it.len - kt * kKTile;  // keys in this tile
#pragma unroll
          for (int qtr = 0; qtr < 4; ++qtr) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int j0 = qtr * 32 + 2 * e;
              pk[e] = j0 + 1 < rem ? 0x3F803F80u : (j0 < rem ? 0x00003F80u : 0u);  // bf16 pairs of 1.0
            }
            tmem_st16(p_addr + qtr * 16, pk);
          }
          row_sum += float(rem < kKTile ? rem : kKTile);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + (P_FULL + w) * 8);
          continue;
        }
        float s2[128];  // raw scores (bias included) of this row against the tile's 128 keys
        tmem_ld32_f128<0>(s_addr, s2);
        tmem_ld32_f128<32>(s_addr + 32, s2);
        tmem_ld32_f128<64>(s_addr + 64, s2);
        tmem_ld32_f128<96>(s_addr + 96, s2);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (S_FREE + w) * 8);  // the S buffer can take the next tile's scores

        const int rem = it.len - kt * kKTile;  // valid keys in this tile
        if (rem < kKTile) {
#pragma unroll
          for (int j = 0; j < 128; ++j)
            if (j >= rem) s2[j] = -INFINITY;
        }
        // The reference point of the exponentials is the maximum of the item's first key tile.  Later tiles
        // skip the search for a maximum: fp32 sums, fp32 O and bf16 P share the fp32 exponent range, so
        // probabilities far above 1 lose nothing, and a tile whose sum leaves the safe range is redone below.
        bool find_anchor = kt == 0;
        if (kMasked) {
          // Keys may be switched off anywhere in the row (the same bits for every query of this item).  A tile
          // without any valid key yields zeros (the reference point stays 0 until a tile with a valid key comes).
          const uint32_t* mrow = p.key_mask + it.b * p.km_b + it.r * p.km_r + kt * 4;
          const int words = (p.S + 31) >> 5;
          uint32_t mw[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) mw[j] = kt * 4 + j < words ? __ldg(mrow + j) : 0u;
#pragma unroll
          for (int j = 0; j < 128; ++j)
            if (!((mw[j >> 5] >> (j & 31)) & 1u)) s2[j] = -INFINITY;
          find_anchor = !have_anchor && (mw[0] | mw[1] | mw[2] | mw[3]) != 0u;
          have_anchor = have_anchor || find_anchor;
        }
        if (kt > 0) {
          // the previous tile's P·V must be complete before P is overwritten
          ok = mbar_wait(bars + (O_FULL + w) * 8, (ct - 1) & 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
        }
        if (find_anchor) {
          float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four independent chains
#pragma unroll
          for (int j = 0; j < 64; ++j) mx[j & 3] = max3_f32(mx[j & 3], s2[2 * j], s2[2 * j + 1]);
          row_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));  // finite: the tile holds a valid key
        }
        // p = 2^(c * (s - row_max)); bf16 pairs go back to TMEM as the A operand of P·V
        float tile_sum;
        {
          const float nmc = -row_max * c;
          const uint64_t nmc2 = pack_f32x2(nmc, nmc);
          uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull};  // four independent packed partial sums
#pragma unroll
          for (int qtr = 0; qtr < 4; ++qtr) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int j0 = qtr * 32 + 2 * e;
              const uint64_t d2 = fma_f32x2(pack_f32x2(s2[j0], s2[j0 + 1]), c2, nmc2);
              float d0, d1;
              unpack_f32x2(d2, d0, d1);
              const uint64_t p2 = pack_f32x2(ex2_approx(d0), ex2_approx(d1));
              sum2[e & 3] = add_f32x2(sum2[e & 3], p2);
              float p0, p1;
              unpack_f32x2(p2, p0, p1);
              pk[e] = pack_bf16x2(p0, p1);
            }
            tmem_st16(p_addr + qtr * 16, pk);
          }
          float a0, a1;
          unpack_f32x2(add_f32x2(add_f32x2(sum2[0], sum2[1]), add_f32x2(sum2[2], sum2[3])), a0, a1);
          tile_sum = a0 + a1;
        }
        // Rare: some score lies so far above the reference point that the tile's sum leaves the safe range (or
        // overflowed).  Move the reference point of the affected rows to the tile's maximum, rescale what has
        // been accumulated (the previous P·V is complete, see above) and redo the tile.
        if (__any_sync(0xffffffffu, !(tile_sum < kRebaseSum))) {
          float cm = -INFINITY;
#pragma unroll
          for (int j = 0; j < 128; ++j) cm = fmaxf(cm, s2[j]);
          const float new_max = (tile_sum < kRebaseSum) ? row_max : cm;
          const float alpha = ex2_approx((row_max - new_max) * c);  // 1 for rows that keep their reference point
          tmem_st_wait();
          if (kt > 0) {
            uint32_t t[32];
            tmem_ld32(o_addr, t);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) t[j] = __float_as_uint(__uint_as_float(t[j]) * alpha);
            tmem_st32(o_addr, t);
          }
          row_sum *= alpha;
          row_max = new_max;
          const float nmc = -row_max * c;
          tile_sum = 0.f;
#pragma unroll
          for (int qtr = 0; qtr < 4; ++qtr) {
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int j0 = qtr * 32 + 2 * e;
              const float p0 = ex2_approx(fmaf(s2[j0], c, nmc)), p1 = ex2_approx(fmaf(s2[j0 + 1], c, nmc));
              tile_sum += p0 + p1;
              pk[e] = pack_bf16x2(p0, p1);
            }
            tmem_st16(p_addr + qtr * 16, pk);
          }
        }
        row_sum += tile_sum;
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (P_FULL + w) * 8);
      }
      if (!ok) break;
      // Output factors first (gate / row sum): they only need the gate row fetched during the last tile, and
      // computing them here fills the time the last P·V takes.
      float sg[32];
      const float inv = 1.f / row_sum;
      if (p.gate != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t gw[4] = {gv[j].x, gv[j].y, gv[j].z, gv[j].w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            sg[j * 8 + 2 * e] = bf16_lo(gw[e]) * inv;
            sg[j * 8 + 2 * e + 1] = bf16_hi(gw[e]) * inv;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) sg[j] = inv;
      }
      // the item's output: O (in TMEM) / row_sum * gate
      ok = mbar_wait(bars + (O_FULL + w) * 8, (ct - 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      uint32_t pk[16];
      {
        uint32_t t[32];
        tmem_ld32(o_addr, t);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          pk[j] = pack_bf16x2(__uint_as_float(t[2 * j]) * sg[2 * j], __uint_as_float(t[2 * j + 1]) * sg[2 * j + 1]);
      }
      tc_fence_before();
      if (q < p.S) {
        if (p.wide_store) {  // two full 32-byte sectors per row instead of four half sectors
          stg256(out_row, pk);
          stg256(out_row + 16, pk + 8);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            reinterpret_cast<uint4*>(out_row)[j] = make_uint4(pk[j * 4], pk[j * 4 + 1], pk[j * 4 + 2], pk[j * 4 + 3]);
        }
        if (p.lse)
          p.lse[((long long)it.br * p.S + q) * kHeads + it.h] =
              it.uniform ? -INFINITY : 0.6931471805599453f * (row_max * c + __log2f(row_sum));
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

namespace b200ta {
namespace {
// Constants for fast_div: with l = ceil(log2 d) and mul = floor(2^(31+l) / d) + 1, floor(n / d) equals
// (n * mul) >> (31 + l) for every n < 2^31.
void fast_div_constants(uint32_t d, uint32_t* mul, uint32_t* shr) {
  if (d <= 1) {
    *mul = 0, *shr = 0;
    return;
  }
  uint32_t l = 0;
  while ((uint64_t(1) << l) < d) ++l;
  *mul = uint32_t((uint64_t(1) << (31 + l)) / d + 1);
  *shr = l - 1;
}
}  // namespace
}  // namespace b200ta

namespace b200ta {
namespace {

int launch_attention(const void* q, const void* k, const void* v, const void* gate, int64_t s_br, int64_t s_h,
                     int64_t s_s, const void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q,
                     const int32_t* lengths, int64_t ls_b, int64_t ls_r, const uint32_t* key_mask, int64_t km_b,
                     int64_t km_r, void* out, int64_t os_br, int64_t os_s, int64_t os_h, float* lse,
                     float softmax_scale, int empty_row_mode, int B, int R, int S, int S_pad, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(q && k && v && bias && out, "attention: NULL pointer");
  B200TA_REQUIRE(B > 0 && R > 0 && S > 0, "attention: bad sizes B=%d R=%d S=%d", B, R, S);
  B200TA_REQUIRE(S_pad >= S && S_pad % 8 == 0, "attention: S_pad=%d must be a multiple of 8 and >= S=%d", S_pad, S);
  B200TA_REQUIRE(softmax_scale > 0.f, "attention: softmax_scale must be positive");
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
  fast_div_constants(uint32_t(R), &p.r_mul, &p.r_shr);
  fast_div_constants(uint32_t(q_pairs), &p.qp_mul, &p.qp_shr);
  p.lengths = lengths;
  p.ls_b = ls_b, p.ls_r = ls_r;
  p.key_mask = key_mask;
  p.km_b = km_b, p.km_r = km_r;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.g_br = s_br, p.g_h = s_h, p.g_s = s_s;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.o_br = os_br, p.o_s = os_s, p.o_h = os_h;
  p.lse = lse;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.empty_uniform = empty_row_mode == B200TA_EMPTY_ROW_UNIFORM ? 1 : 0;
  p.wide_store = (reinterpret_cast<uintptr_t>(out) & 31u) == 0 && os_br % 16 == 0 && os_s % 16 == 0 && os_h % 16 == 0;
  p.status = st->status_dev;

  const int grid = p.num_items < st->num_sms ? p.num_items : st->num_sms;
  if (key_mask != nullptr) {
    B200TA_REQUIRE(lengths != nullptr, "attention: the masked form needs the row lengths (last valid key + 1) as well");
    B200TA_CHECK_CUDA(cudaFuncSetAttribute(attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
    attention_kernel<true><<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, tm_bias, p);
  } else {
    B200TA_CHECK_CUDA(cudaFuncSetAttribute(attention_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmDynamic));
    attention_kernel<false><<<grid, kThreads, kSmDynamic, static_cast<cudaStream_t>(stream)>>>(tm_q, tm_k, tm_v, tm_bias, p);
  }
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_attention(const void* q, const void* k, const void* v, const void* gate, int64_t s_br, int64_t s_h,
                     int64_t s_s, const void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q,
                     const int32_t* lengths, int64_t ls_b, int64_t ls_r, void* out, int64_t os_br, int64_t os_s,
                     int64_t os_h, float* lse, float softmax_scale, int empty_row_mode, int B, int R, int S,
                     int S_pad, void* stream) {
  return b200ta::launch_attention(q, k, v, gate, s_br, s_h, s_s, bias, bs_b, bs_h, bs_q, lengths, ls_b, ls_r, nullptr, 0,
                                  0, out, os_br, os_s, os_h, lse, softmax_scale, empty_row_mode, B, R, S, S_pad, stream);
}

int b200ta_attention_masked(const void* q, const void* k, const void* v, const void* gate, int64_t s_br, int64_t s_h,
                            int64_t s_s, const void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q,
                            const int32_t* lengths, int64_t ls_b, int64_t ls_r, const uint32_t* key_mask,
                            int64_t km_b, int64_t km_r, void* out, int64_t os_br, int64_t os_s, int64_t os_h,
                            float* lse, float softmax_scale, int empty_row_mode, int B, int R, int S, int S_pad,
                            void* stream) {
  if (key_mask == nullptr) return b200ta::fail(B200TA_ERR_INVALID, "attention_masked: key_mask must not be NULL");
  return b200ta::launch_attention(q, k, v, gate, s_br, s_h, s_s, bias, bs_b, bs_h, bs_q, lengths, ls_b, ls_r, key_mask,
                                  km_b, km_r, out, os_br, os_s, os_h, lse, softmax_scale, empty_row_mode, B, R, S, S_pad,
                                  stream);
}

}  // extern "C"
