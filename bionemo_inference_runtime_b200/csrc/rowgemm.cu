// Row-tile GEMM kernels of the triangle-attention node (sm_100a).
//
// One persistent CTA per SM walks 128-position tiles of the pair tensor.  For each tile the 128x128 bf16
// activation block arrives by TMA as the K-major A operand, the weights (resident in shared memory for the
// whole kernel) are the B operand, tcgen05.mma accumulates into TMEM and eight epilogue warps (one TMEM lane =
// one position = one thread per warpgroup, the two warpgroups take alternate 32-column groups) finish the rows
// and store them with 32-byte vector stores where alignment allows (64 contiguous bytes per thread and group).
//
//   kPrologue: z tile -> LayerNorm statistics (from the smem copy) while the tensor core multiplies the raw
//              rows with the LayerNorm-folded weights: q,k,v,g (512 columns, written head-major; the g plane
//              as sigmoid(g)) and 4 triangle-bias heads.
//   kEpilogue: og tile -> og · W_oᵀ + b_o + residual.
//
// Warp roles (320 threads): warps 0-7 epilogue (TMEM lanes 32(w%4)..+31), warp 8 TMA producer, warp 9 MMA
// issuer / TMEM owner.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr int kTileM = 128;
constexpr int kThreads = 320;
constexpr int kSlotCols = 256;  // TMEM columns per accumulator slot (2 slots)

enum Mode { kPrologue = 0, kEpilogue = 1 };
constexpr int kMaxPeers = 8;

struct RowGemmParams {
  int B, R, S, S_pad;
  int tiles_s;
  int num_tiles;
  const float2* sc;  // prologue: {rowsum, const} per folded row
  const float* bo;   // epilogue: output bias
  const int* flags;  // prologue: flags[0] != 0 -> apply LayerNorm statistics
  float eps;
  __nv_bfloat16* bias;
  long long bs_b, bs_h, bs_q, bs_k;
  __nv_bfloat16* out;                         // prologue: q/k/v/g planes; epilogue: output pair tensor
  long long qs_which, qs_br, qs_h, qs_s;      // prologue strides (elements)
  long long os_b, os_r, os_s;                 // epilogue strides (elements)
  // epilogue, transposing mode (num_peers > 0): position (b, r, s) goes to the column shard of GPU s / peer_cols,
  // a [B][peer_rows][peer_cols][128] tensor, at (b, row0 + r, s % peer_cols)
  __nv_bfloat16* peers[kMaxPeers];
  int num_peers, peer_cols, peer_rows, row0;
  int want_qkvg;
  int has_residual;
  int wide_store;  // output base 32-byte aligned and every stride a multiple of 16 elements
  int* status;
};

template <int MODE>
struct Smem {
  static constexpr int kWRows = MODE == kPrologue ? kNodeRows : kC;
  static constexpr int kWHalf = kWRows * 128;  // bytes of one 64-channel half
  static constexpr int kW = 0;
  static constexpr int kA = kW + 2 * kWHalf;   // 2 stages x 32 KiB
  static constexpr int kRes = kA + 2 * 32768;  // epilogue only: 2 stages x 32 KiB
  static constexpr int kVec = kRes + (MODE == kEpilogue ? 2 * 32768 : 0);
  // prologue: per column pair {rowsum0, rowsum1, const0, const1}; epilogue: b_o
  static constexpr int kVecBytes = MODE == kPrologue ? (kNodeRows / 2) * 16 : kC * 4;
  static constexpr int kBars = kVec + kVecBytes;
  static constexpr int kTotal = kBars + 128;
  static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
};

// barrier slots inside the kBars block (8 bytes each)
enum Bar { W_FULL = 0, A_FULL = 1, A_EMPTY = 3, ACC_FULL = 5, ACC_EMPTY = 7, NUM_BARS = 9 };

__device__ __forceinline__ void stg128(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  *reinterpret_cast<uint4*>(p) = make_uint4(a, b, c, d);
}
// 32-byte store (one full sector per lane); the address must be 32-byte aligned.
__device__ __forceinline__ void stg256(void* p, const uint32_t* v) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
               "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}

// 64 contiguous bytes of one output row: two 32-byte stores when base and strides allow, else four of 16.
__device__ __forceinline__ void store_row64(__nv_bfloat16* dst, const uint32_t (&v)[16], bool wide) {
  if (wide) {
    stg256(dst, v);
    stg256(dst + 16, v + 8);
  } else {
#pragma unroll
    for (int c = 0; c < 4; ++c) stg128(dst + c * 8, v[c * 4], v[c * 4 + 1], v[c * 4 + 2], v[c * 4 + 3]);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
rowgemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_w,
               const __grid_constant__ CUtensorMap tm_res, const RowGemmParams p) {
  using L = Smem<MODE>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));  // generic pointer to the aligned base
  const uint32_t bars = base + L::kBars;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(gen + L::kBars + NUM_BARS * 8 + 8);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(gen + L::kBars + NUM_BARS * 8);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int u_begin = (MODE == kPrologue && !p.want_qkvg) ? 2 : 0;
  const int u_end = MODE == kPrologue ? 3 : 1;

  if (threadIdx.x == 0) {
    abort_flag[0] = 0;
    abort_flag[1] = 0;  // scratch flag for the producer's drain wait
    mbar_init(bars + W_FULL * 8, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bars + (A_FULL + i) * 8, 1);
      mbar_init(bars + (A_EMPTY + i) * 8, 9);  // 8 epilogue warps + the MMA commit
      mbar_init(bars + (ACC_FULL + i) * 8, 1);
      mbar_init(bars + (ACC_EMPTY + i) * 8, 8);
    }
    fence_mbar_init();
  }
  // stage the per-column vectors
  if (MODE == kPrologue) {
    float4* dst = reinterpret_cast<float4*>(gen + L::kVec);
    for (int i = threadIdx.x; i < kNodeRows / 2; i += kThreads) {
      const float2 a = p.sc[2 * i], b = p.sc[2 * i + 1];
      dst[i] = make_float4(a.x, b.x, a.y, b.y);
    }
  } else {
    float* dst = reinterpret_cast<float*>(gen + L::kVec);
    for (int i = threadIdx.x; i < kC; i += kThreads) dst[i] = p.bo[i];
  }
  if (warp == 9) tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int my_tiles = (p.num_tiles - 1 - int(blockIdx.x)) / int(gridDim.x) + 1;  // blockIdx.x < num_tiles

  if (warp == 8) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_a);
      tma_prefetch_desc(&tm_w);
      mbar_expect_tx(bars + W_FULL * 8, 2 * L::kWHalf);
      constexpr int kBoxRows = MODE == kPrologue ? 176 : 128;
      for (int kh = 0; kh < 2; ++kh)
        for (int j = 0; j < L::kWRows / kBoxRows; ++j)
          tma_load_2d(base + L::kW + kh * L::kWHalf + j * kBoxRows * 128, &tm_w, bars + W_FULL * 8, kh * 64,
                      j * kBoxRows);
      int issued = 0;
      for (int i = 0; i < my_tiles; ++i) {
        const int tile = blockIdx.x + i * gridDim.x;
        const int st = tile % p.tiles_s;
        const int br = tile / p.tiles_s;
        const int r = br % p.R, b = br / p.R;
        const int stage = i & 1;
        if (!mbar_wait(bars + (A_EMPTY + stage) * 8, ((i >> 1) & 1) ^ 1, abort_flag)) break;
        const uint32_t full = bars + (A_FULL + stage) * 8;
        const bool with_res = MODE == kEpilogue && p.has_residual;
        mbar_expect_tx(full, 32768 + (with_res ? 32768 : 0));
        tma_load_4d(base + L::kA + stage * 32768, &tm_a, full, 0, st * kTileM, r, b);
        tma_load_4d(base + L::kA + stage * 32768 + 16384, &tm_a, full, 64, st * kTileM, r, b);
        if (with_res)
          for (int g = 0; g < 4; ++g)
            tma_load_4d(base + L::kRes + stage * 32768 + g * 8192, &tm_res, full, g * 32, st * kTileM, r, b);
        ++issued;
      }
      // If the loop was abandoned, give copies still in flight a bounded chance to land.
      if (*abort_flag && issued > 0) {
        const int last = issued - 1;
        mbar_wait(bars + (A_FULL + (last & 1)) * 8, (last >> 1) & 1, abort_flag + 1);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      bool ok = mbar_wait(bars + W_FULL * 8, 0, abort_flag);
      int uc = 0;  // accumulator-slot use counter
      for (int i = 0; ok && i < my_tiles; ++i) {
        const int stage = i & 1;
        ok = mbar_wait(bars + (A_FULL + stage) * 8, (i >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int u = u_begin; u < u_end; ++u, ++uc) {
          const int slot = uc & 1;
          ok = mbar_wait(bars + (ACC_EMPTY + slot) * 8, ((uc >> 1) & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const int n = MODE == kEpilogue ? 128 : (u < 2 ? 256 : 16);
          const uint32_t idesc = make_idesc_bf16(kTileM, n);
          const uint32_t d = tmem_base + slot * kSlotCols;
          // one descriptor per operand; each K step adds a constant to the address field (16-byte units)
          const uint64_t da = make_smem_desc(base + L::kA + stage * 32768, 16, 1024, kLayoutSw128);
          const uint64_t db = make_smem_desc(base + L::kW + u * 256 * 128, 16, 1024, kLayoutSw128);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            umma_ss(d, da + ((k >> 2) * (16384 >> 4) + (k & 3) * 2), db + ((k >> 2) * (L::kWHalf >> 4) + (k & 3) * 2),
                    idesc, k > 0 ? 1u : 0u);
          umma_commit(bars + (ACC_FULL + slot) * 8);
        }
        if (!ok) break;
        umma_commit(bars + (A_EMPTY + stage) * 8);
      }
    }
  } else {
    // ------------------------------------------------------------- epilogue warps
    const int e = warp >> 2;               // which alternate column groups this warpgroup takes
    const int m = (warp & 3) * 32 + lane;  // row of the tile == TMEM lane
    const uint32_t lane_taddr = tmem_base + (uint32_t((warp & 3) * 32) << 16);
    const bool normalize = MODE == kPrologue && __ldg(p.flags) != 0;
    int uc = 0;
    bool ok = true;
    for (int i = 0; ok && i < my_tiles; ++i) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int st = tile % p.tiles_s;
      const int br = tile / p.tiles_s;
      const int r = br % p.R, b = br / p.R;
      const int stage = i & 1;
      const int s = st * kTileM + m;  // this thread's position along the sequence axis
      ok = mbar_wait(bars + (A_FULL + stage) * 8, (i >> 1) & 1, abort_flag);
      if (!ok) break;
      float rstd = 1.f, nmr = 0.f;
      if (normalize) {
        // LayerNorm statistics of row m from the swizzled smem copy of the z tile.
        uint32_t v[64];
        const uint32_t a0 = base + L::kA + stage * 32768;
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
      if (MODE == kPrologue) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (A_EMPTY + stage) * 8);  // done reading the z tile
      }
      const uint64_t rstd2 = pack_f32x2(rstd, rstd), nmr2 = pack_f32x2(nmr, nmr);
      for (int u = u_begin; ok && u < u_end; ++u, ++uc) {
        const int slot = uc & 1;
        ok = mbar_wait(bars + (ACC_FULL + slot) * 8, (uc >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc_addr = lane_taddr + slot * kSlotCols;
        if (MODE == kPrologue && u == 2) {
          // triangle-bias heads: columns 512..515 of the folded projection (first warpgroup only)
          if (e == 0) {
            uint32_t a[16];
            tmem_ld16(acc_addr, a);
            tmem_ld_wait();
            const float4* sc4 = reinterpret_cast<const float4*>(gen + L::kVec) + 256;
            if (p.bias != nullptr && s < p.S_pad) {
#pragma unroll
              for (int hp = 0; hp < 2; ++hp) {
                const float4 t = sc4[hp];  // {rowsum0, rowsum1, const0, const1}
                const float v0 = s < p.S ? fmaf(rstd, __uint_as_float(a[2 * hp]), fmaf(nmr, t.x, t.z)) : 0.f;
                const float v1 = s < p.S ? fmaf(rstd, __uint_as_float(a[2 * hp + 1]), fmaf(nmr, t.y, t.w)) : 0.f;
                p.bias[b * p.bs_b + (2 * hp) * p.bs_h + r * p.bs_q + s * p.bs_k] = __float2bfloat16_rn(v0);
                p.bias[b * p.bs_b + (2 * hp + 1) * p.bs_h + r * p.bs_q + s * p.bs_k] = __float2bfloat16_rn(v1);
              }
            }
          }
        } else {
          // This warpgroup takes the 32-column groups e, e+2, ...  The TMEM load of the next group is issued
          // before the current group's math, and the per-column constants are fetched from shared memory
          // before the wait for the current load, so neither latency is exposed.
          constexpr int kGroupsPerWg = MODE == kPrologue ? 4 : 2;
          uint32_t acc[2][32];
          tmem_ld32(acc_addr + e * 32, acc[0]);
#pragma unroll
          for (int gi = 0; gi < kGroupsPerWg; ++gi) {
            const int g = e + 2 * gi;
            const int n0 = (MODE == kPrologue ? u * 256 : 0) + g * 32;
            uint32_t (&a)[32] = acc[gi & 1];
            uint32_t packed[16];
            if (MODE == kPrologue) {
              float4 t[16];  // {rowsum0, rowsum1, const0, const1} of columns n0+2j, n0+2j+1
              const float4* sc4 = reinterpret_cast<const float4*>(gen + L::kVec) + (n0 >> 1);
#pragma unroll
              for (int j = 0; j < 16; ++j) t[j] = sc4[j];
              tmem_ld_wait();
              if (gi + 1 < kGroupsPerWg) tmem_ld32(acc_addr + (g + 2) * 32, acc[(gi + 1) & 1]);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const uint64_t off = fma_f32x2(nmr2, pack_f32x2(t[j].x, t[j].y), pack_f32x2(t[j].z, t[j].w));
                float o0, o1;
                unpack_f32x2(fma_f32x2(rstd2, pack_f32x2(__uint_as_float(a[2 * j]), __uint_as_float(a[2 * j + 1])), off),
                             o0, o1);
                packed[j] = pack_bf16x2(o0, o1);
              }
              if (n0 >= 3 * kC) {
                // Gate plane: store sigmoid(g), computed from the bf16-rounded logit and rounded to bf16 again
                // as the eager bf16 module does (gate.sigmoid_() on a bf16 tensor).  The attention kernel then
                // only multiplies.  sigmoid(x) = 0.5 * tanh(x / 2) + 0.5.
#pragma unroll
                for (int j = 0; j < 16; ++j)
                  packed[j] = pack_bf16x2(fmaf(0.5f, tanh_approx(0.5f * bf16_lo(packed[j])), 0.5f),
                                          fmaf(0.5f, tanh_approx(0.5f * bf16_hi(packed[j])), 0.5f));
              }
              if (s < p.S) {
                // head-major planes: 64 contiguous bytes per (plane, head, position)
                __nv_bfloat16* dst = p.out + (n0 >> 7) * p.qs_which + (long long)br * p.qs_br + ((n0 >> 5) & 3) * p.qs_h +
                                     (long long)s * p.qs_s;
                store_row64(dst, packed, p.wide_store != 0);
              }
            } else {
              const float* bo = reinterpret_cast<const float*>(gen + L::kVec) + n0;
              uint32_t res[16];
              if (p.has_residual) {
                const uint32_t r0 = base + L::kRes + stage * 32768 + g * 8192;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  uint4 x = lds128(r0 + sw64_offset(m, c));
                  res[c * 4 + 0] = x.x, res[c * 4 + 1] = x.y, res[c * 4 + 2] = x.z, res[c * 4 + 3] = x.w;
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) res[j] = 0u;
              }
              float bov[32];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 t = reinterpret_cast<const float4*>(bo)[j];
                bov[4 * j] = t.x, bov[4 * j + 1] = t.y, bov[4 * j + 2] = t.z, bov[4 * j + 3] = t.w;
              }
              tmem_ld_wait();
              if (gi + 1 < kGroupsPerWg) tmem_ld32(acc_addr + (g + 2) * 32, acc[(gi + 1) & 1]);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float o0 = __uint_as_float(a[2 * j]) + bov[2 * j] + bf16_lo(res[j]);
                const float o1 = __uint_as_float(a[2 * j + 1]) + bov[2 * j + 1] + bf16_hi(res[j]);
                packed[j] = pack_bf16x2(o0, o1);
              }
              if (s < p.S) {
                __nv_bfloat16* dst;
                if (p.num_peers > 0) {
                  const int peer = s / p.peer_cols;
                  dst = p.peers[peer] +
                        (((long long)b * p.peer_rows + p.row0 + r) * p.peer_cols + (s - peer * p.peer_cols)) * kC + n0;
                } else {
                  dst = p.out + b * p.os_b + r * p.os_r + (long long)s * p.os_s + n0;
                }
                store_row64(dst, packed, p.wide_store != 0);
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (ACC_EMPTY + slot) * 8);
      }
      if (MODE == kEpilogue) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + (A_EMPTY + stage) * 8);  // done reading the residual tile
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_flag) *p.status = B200TA_ERR_DEVICE_WAIT;
}

int check_strides(const char* what, int64_t s0, int64_t s1, int64_t s2) {
  if (s0 % 8 != 0 || s1 % 8 != 0 || s2 % 8 != 0 || s0 < 0 || s1 < 0 || s2 < 0)
    return fail(B200TA_ERR_INVALID, "%s: element strides must be non-negative multiples of 8 (16 bytes)", what);
  return B200TA_OK;
}

// 4-D map over a pair tensor [B,R,S,128]: dims (c, s, r, b).
int pair_tensor_map(CUtensorMap* map, const void* ptr, int64_t sb, int64_t sr, int64_t ss, int B, int R, int S,
                    uint32_t box_c, uint32_t box_s, SwizzleMode swz, const char* what) {
  // A size-1 dimension may carry any stride; give it a valid one.
  auto fix = [](int64_t stride, int extent) -> uint64_t { return extent == 1 ? 256u : uint64_t(stride) * 2u; };
  uint64_t dims[4] = {uint64_t(kC), uint64_t(S), uint64_t(R), uint64_t(B)};
  uint64_t strides[3] = {fix(ss, S), fix(sr, R), fix(sb, B)};
  uint32_t box[4] = {box_c, box_s, 1, 1};
  return encode_tensor_map(map, ptr, 2, 4, dims, strides, box, swz, what);
}

// Shared by the two epilogue entry points: `p` arrives with its output addressing filled in.
int launch_epilogue(const void* og, int64_t gs_b, int64_t gs_r, int64_t gs_s, const void* packed, const void* residual,
                    int64_t rs_b, int64_t rs_r, int64_t rs_s, RowGemmParams p, int B, int R, int S, void* stream) {
  B200TA_REQUIRE(og && packed, "epilogue: NULL pointer");
  B200TA_REQUIRE(B > 0 && R > 0 && S > 0, "epilogue: bad sizes B=%d R=%d S=%d", B, R, S);
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "epilogue: packed must be 256-byte aligned");
  int rc = check_strides("epilogue og", gs_b, gs_r, gs_s);
  if (rc == B200TA_OK && residual) rc = check_strides("epilogue residual", rs_b, rs_r, rs_s);
  if (rc != B200TA_OK) return rc;
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  CUtensorMap tm_a, tm_w, tm_res;
  rc = pair_tensor_map(&tm_a, og, gs_b, gs_r, gs_s, B, R, S, 64, kTileM, SWZ_128, "epilogue og");
  if (rc != B200TA_OK) return rc;
  const char* pk = static_cast<const char*>(packed);
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(kC)};
    uint64_t strides[1] = {uint64_t(kC) * 2};
    uint32_t box[2] = {64, 128};
    rc = encode_tensor_map(&tm_w, pk + kNodeWoOff, 2, 2, dims, strides, box, SWZ_128, "epilogue weights");
    if (rc != B200TA_OK) return rc;
  }
  if (residual) {
    rc = pair_tensor_map(&tm_res, residual, rs_b, rs_r, rs_s, B, R, S, 32, kTileM, SWZ_64, "epilogue residual");
    if (rc != B200TA_OK) return rc;
  } else {
    tm_res = tm_a;
  }
  p.B = B, p.R = R, p.S = S, p.S_pad = S;
  p.tiles_s = (S + kTileM - 1) / kTileM;
  p.num_tiles = B * R * p.tiles_s;
  p.bo = reinterpret_cast<const float*>(pk + kNodeBoOff);
  p.flags = reinterpret_cast<const int*>(pk + kNodeFlagsOff);
  p.has_residual = residual ? 1 : 0;
  p.status = st->status_dev;

  auto kern = rowgemm_kernel<kEpilogue>;
  B200TA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<kEpilogue>::kDynamic));
  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  kern<<<grid, kThreads, Smem<kEpilogue>::kDynamic, static_cast<cudaStream_t>(stream)>>>(tm_a, tm_w, tm_res, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_prologue(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed, float eps,
                    void* qkvg, int64_t qs_which, int64_t qs_br, int64_t qs_h, int64_t qs_s, int want_qkvg,
                    void* bias, int64_t bs_b, int64_t bs_h, int64_t bs_q, int64_t bs_k, int B, int R, int S,
                    int S_pad, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(z && packed, "prologue: NULL pointer");
  B200TA_REQUIRE(B > 0 && R > 0 && S > 0 && S_pad >= S, "prologue: bad sizes B=%d R=%d S=%d S_pad=%d", B, R, S, S_pad);
  B200TA_REQUIRE(want_qkvg ? qkvg != nullptr : bias != nullptr, "prologue: nothing to write");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "prologue: packed must be 256-byte aligned");
  B200TA_REQUIRE(int64_t(B) * R < (int64_t(1) << 31), "prologue: B*R too large");
  int rc = check_strides("prologue z", zs_b, zs_r, zs_s);
  if (rc != B200TA_OK) return rc;
  if (want_qkvg) {
    rc = check_strides("prologue qkvg", qs_which, qs_br, qs_h);
    if (rc != B200TA_OK) return rc;
    B200TA_REQUIRE(qs_s % 8 == 0 && qs_s > 0, "prologue qkvg: s stride must be a positive multiple of 8");
    B200TA_REQUIRE((reinterpret_cast<uintptr_t>(qkvg) & 15u) == 0, "prologue: qkvg must be 16-byte aligned");
  }
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != B200TA_OK) return rc;

  CUtensorMap tm_a, tm_w;
  rc = pair_tensor_map(&tm_a, z, zs_b, zs_r, zs_s, B, R, S, 64, kTileM, SWZ_128, "prologue z");
  if (rc != B200TA_OK) return rc;
  const char* pk = static_cast<const char*>(packed);
  {
    uint64_t dims[2] = {uint64_t(kC), uint64_t(kNodeRows)};
    uint64_t strides[1] = {uint64_t(kC) * 2};
    uint32_t box[2] = {64, 176};
    rc = encode_tensor_map(&tm_w, pk + kNodeWOff, 2, 2, dims, strides, box, SWZ_128, "prologue weights");
    if (rc != B200TA_OK) return rc;
  }

  RowGemmParams p{};
  p.B = B, p.R = R, p.S = S, p.S_pad = S_pad;
  p.tiles_s = (S + kTileM - 1) / kTileM;
  p.num_tiles = B * R * p.tiles_s;
  p.sc = reinterpret_cast<const float2*>(pk + kNodeScOff);
  p.flags = reinterpret_cast<const int*>(pk + kNodeFlagsOff);
  p.eps = eps;
  p.bias = static_cast<__nv_bfloat16*>(bias);
  p.bs_b = bs_b, p.bs_h = bs_h, p.bs_q = bs_q, p.bs_k = bs_k;
  p.out = static_cast<__nv_bfloat16*>(qkvg);
  p.qs_which = qs_which, p.qs_br = qs_br, p.qs_h = qs_h, p.qs_s = qs_s;
  p.want_qkvg = want_qkvg ? 1 : 0;
  p.wide_store = (reinterpret_cast<uintptr_t>(qkvg) & 31u) == 0 && qs_which % 16 == 0 && qs_br % 16 == 0 &&
                 qs_h % 16 == 0 && qs_s % 16 == 0;
  p.status = st->status_dev;

  auto kern = rowgemm_kernel<kPrologue>;
  B200TA_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<kPrologue>::kDynamic));
  const int grid = p.num_tiles < st->num_sms ? p.num_tiles : st->num_sms;
  kern<<<grid, kThreads, Smem<kPrologue>::kDynamic, static_cast<cudaStream_t>(stream)>>>(tm_a, tm_w, tm_a, p);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

int b200ta_epilogue(const void* og, int64_t gs_b, int64_t gs_r, int64_t gs_s, const void* packed,
                    const void* residual, int64_t rs_b, int64_t rs_r, int64_t rs_s, void* out, int64_t os_b,
                    int64_t os_r, int64_t os_s, int B, int R, int S, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(out, "epilogue: NULL pointer");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(out) & 15u) == 0, "epilogue: out must be 16-byte aligned");
  int rc = check_strides("epilogue out", os_b, os_r, os_s);
  if (rc != B200TA_OK) return rc;
  RowGemmParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.os_b = os_b, p.os_r = os_r, p.os_s = os_s;
  p.wide_store = (reinterpret_cast<uintptr_t>(out) & 31u) == 0 && os_b % 16 == 0 && os_r % 16 == 0 && os_s % 16 == 0;
  return launch_epilogue(og, gs_b, gs_r, gs_s, packed, residual, rs_b, rs_r, rs_s, p, B, R, S, stream);
}

int b200ta_epilogue_scatter(const void* og, int64_t gs_b, int64_t gs_r, int64_t gs_s, const void* packed,
                            const void* residual, int64_t rs_b, int64_t rs_r, int64_t rs_s, void* const* peer_out,
                            int num_peers, int rank, int B, int R, int S, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(peer_out, "epilogue_scatter: NULL pointer");
  B200TA_REQUIRE(num_peers >= 1 && num_peers <= kMaxPeers && rank >= 0 && rank < num_peers,
                 "epilogue_scatter: need 1..%d peers and 0 <= rank < peers, got %d and %d", kMaxPeers, num_peers, rank);
  B200TA_REQUIRE(S % num_peers == 0 && R == S / num_peers,
                 "epilogue_scatter: S=%d must be divisible by the %d peers and R=%d must equal S / peers", S, num_peers, R);
  RowGemmParams p{};
  for (int g = 0; g < num_peers; ++g) {
    B200TA_REQUIRE(peer_out[g] && (reinterpret_cast<uintptr_t>(peer_out[g]) & 31u) == 0,
                   "epilogue_scatter: peer buffer %d must be a 32-byte aligned device pointer", g);
    p.peers[g] = static_cast<__nv_bfloat16*>(peer_out[g]);
  }
  p.num_peers = num_peers, p.peer_cols = R, p.peer_rows = S, p.row0 = rank * R;
  p.wide_store = 1;
  return launch_epilogue(og, gs_b, gs_r, gs_s, packed, residual, rs_b, rs_r, rs_s, p, B, R, S, stream);
}

}  // extern "C"
