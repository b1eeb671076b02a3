// Weight packing: folds LayerNorm's affine into the linear layer that follows it.
//
// For a row w of a projection applied to LN(z) = (z - mu) * rstd * gamma + beta:
//   proj = rstd * sum_c (z_c - mu) * (gamma_c * w_c)  +  sum_c beta_c * w_c  + b
// Subtracting the mean of (gamma*w) from the row leaves the first sum unchanged
// (sum_c (z_c - mu) = 0), and keeps the tensor-core dot product of raw z rows with
// the folded row free of a large common-mode term.  The bf16 rounding of the
// centred row makes its sum slightly non-zero; that sum is stored so the GEMM
// epilogue can subtract mu * rowsum exactly:
//   proj = rstd * (acc - mu * rowsum) + const.
#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

__device__ __forceinline__ float load_w(const void* p, int dtype, size_t i) {
  return dtype == B200TA_DTYPE_F32 ? reinterpret_cast<const float*>(p)[i]
                                   : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// One block of 128 threads per output row.  Rows [0, rows_a) come from `wa`, rows
// [rows_a, rows_a + rows_b) from `wb`, the rest are zero.  Rows in
// [scale_from, scale_to) are multiplied by `scale` (constant term included).
__global__ void fold_rows_kernel(const void* wa, int rows_a, const void* wb, int rows_b,
                                 const void* bias_a, const void* gamma, const void* beta, int dtype,
                                 int scale_from, int scale_to, float scale, __nv_bfloat16* wp,
                                 float2* sc, int* flags) {
  const int n = blockIdx.x;
  const int c = threadIdx.x;
  __shared__ float red[3][4];
  float w = 0.f, b = 0.f;
  if (n < rows_a) {
    if (wa != nullptr) w = load_w(wa, dtype, size_t(n) * kC + c);
    if (bias_a != nullptr) b = load_w(bias_a, dtype, n);
  } else if (n < rows_a + rows_b) {
    w = load_w(wb, dtype, size_t(n - rows_a) * kC + c);
  }
  const float s = (n >= scale_from && n < scale_to) ? scale : 1.f;
  w *= s;
  b *= s;
  // gamma == NULL: the input is already normalised; plain projection, no centring
  const bool normalize = gamma != nullptr;
  const float g = normalize ? load_w(gamma, dtype, c) : 1.f;
  const float be = normalize ? load_w(beta, dtype, c) : 0.f;
  if (n == 0 && c == 0) flags[0] = normalize ? 1 : 0;
  float wg = w * g;
  float cterm = w * be;
  // block reductions over the 128 channels
  auto block_sum = [&](float v, int slot) -> float {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) red[slot][threadIdx.x >> 5] = v;
    __syncthreads();
    return red[slot][0] + red[slot][1] + red[slot][2] + red[slot][3];
  };
  const float mean = normalize ? block_sum(wg, 0) * (1.f / kC) : 0.f;
  const float csum = block_sum(cterm, 1);
  const __nv_bfloat16 q = __float2bfloat16_rn(wg - mean);
  wp[size_t(n) * kC + c] = q;
  const float rowsum = block_sum(__bfloat162float(q), 2);
  if (c == 0) sc[n] = make_float2(rowsum, csum + b);
}

__global__ void convert_kernel(const void* src, int dtype, size_t n, __nv_bfloat16* dst_bf16,
                               float* dst_f32) {
  size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = src == nullptr ? 0.f : load_w(src, dtype, i);
  if (dst_bf16 != nullptr) dst_bf16[i] = __float2bfloat16_rn(v);
  if (dst_f32 != nullptr) dst_f32[i] = v;
}

__global__ void set_flag_kernel(int* flags, int value) { flags[0] = value; }

// The transition's LayerNorm vectors as floats (gamma | beta) and its "apply the LayerNorm" flag.
void pack_transition_layernorm(const void* ln_w, const void* ln_b, int dtype, char* base, cudaStream_t s) {
  float* ln = reinterpret_cast<float*>(base + kTransLnOff);
  convert_kernel<<<1, kC, 0, s>>>(ln_w, dtype, kC, nullptr, ln);
  convert_kernel<<<1, kC, 0, s>>>(ln_b, dtype, kC, nullptr, ln + kC);
  set_flag_kernel<<<1, 1, 0, s>>>(reinterpret_cast<int*>(base + kTransFlagsOff), ln_w != nullptr ? 1 : 0);
}

int check_dtype(int dtype) {
  if (dtype != B200TA_DTYPE_BF16 && dtype != B200TA_DTYPE_F32)
    return fail(B200TA_ERR_INVALID, "weight_dtype must be B200TA_DTYPE_BF16 or B200TA_DTYPE_F32");
  return B200TA_OK;
}

}  // namespace
}  // namespace b200ta

extern "C" {

size_t b200ta_node_pack_bytes(void) { return b200ta::kNodePackBytes; }
size_t b200ta_transition_pack_bytes(void) { return b200ta::kTransPackBytes; }

int b200ta_pack_node_weights(const void* ln_w, const void* ln_b, const void* w_in, const void* b_in,
                             const void* w_bias, const void* w_out, const void* b_out,
                             int weight_dtype, void* packed, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(w_in && w_bias && w_out && packed, "pack_node_weights: NULL pointer");
  B200TA_REQUIRE((ln_w == nullptr) == (ln_b == nullptr), "pack_node_weights: pass both LayerNorm vectors or neither");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "pack_node_weights: packed must be 256-byte aligned");
  int rc = check_dtype(weight_dtype);
  if (rc != B200TA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(packed);
  // the attention kernel adds the bias to q·k before the softmax scale: store bias / scale = bias * sqrt(head_dim)
  constexpr float kBiasScale = 5.656854249492381f;
  fold_rows_kernel<<<kNodeRows, kC, 0, s>>>(
      w_in, 4 * kHeads * kHeadDim, w_bias, kHeads, b_in, ln_w, ln_b, weight_dtype, 4 * kHeads * kHeadDim,
      4 * kHeads * kHeadDim + kHeads, kBiasScale, reinterpret_cast<__nv_bfloat16*>(base + kNodeWOff),
      reinterpret_cast<float2*>(base + kNodeScOff), reinterpret_cast<int*>(base + kNodeFlagsOff));
  convert_kernel<<<(kC * kC + 255) / 256, 256, 0, s>>>(w_out, weight_dtype, size_t(kC) * kC,
                                                       reinterpret_cast<__nv_bfloat16*>(base + kNodeWoOff), nullptr);
  convert_kernel<<<1, kC, 0, s>>>(b_out, weight_dtype, kC, nullptr, reinterpret_cast<float*>(base + kNodeBoOff));
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

int b200ta_pack_pair_bias_weights(const void* ln_w, const void* ln_b, const void* w_z, int num_heads,
                                  float bias_scale, int weight_dtype, void* packed, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(w_z && packed, "pack_pair_bias_weights: NULL pointer");
  B200TA_REQUIRE(num_heads > 0 && num_heads <= 16, "pack_pair_bias_weights: num_heads=%d must be 1..16", num_heads);
  B200TA_REQUIRE((ln_w == nullptr) == (ln_b == nullptr), "pack_pair_bias_weights: pass both LayerNorm vectors or neither");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "pack_pair_bias_weights: packed must be 256-byte aligned");
  int rc = check_dtype(weight_dtype);
  if (rc != B200TA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(packed);
  B200TA_CHECK_CUDA(cudaMemsetAsync(base, 0, kNodePackBytes, s));
  // rows 0..511 (q, k, v, g of a triangle node) stay zero; the bias heads follow
  constexpr int kFirst = 4 * kHeads * kHeadDim;
  fold_rows_kernel<<<kNodeRows, kC, 0, s>>>(
      nullptr, kFirst, w_z, num_heads, nullptr, ln_w, ln_b, weight_dtype, kFirst, kFirst + num_heads, bias_scale,
      reinterpret_cast<__nv_bfloat16*>(base + kNodeWOff), reinterpret_cast<float2*>(base + kNodeScOff),
      reinterpret_cast<int*>(base + kNodeFlagsOff));
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

size_t b200ta_trimul_pack_bytes(void) { return b200ta::kTriPackBytes; }

int b200ta_pack_trimul_weights(const void* ln_in_w, const void* ln_in_b, const void* w_p_in, const void* b_p_in,
                               const void* w_g_in, const void* b_g_in, const void* ln_out_w, const void* ln_out_b,
                               const void* w_p_out, const void* b_p_out, const void* w_g_out, const void* b_g_out,
                               int weight_dtype, void* packed, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(ln_in_w && ln_in_b && w_p_in && w_g_in && ln_out_w && ln_out_b && w_p_out && w_g_out && packed,
                 "pack_trimul_weights: NULL pointer");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "pack_trimul_weights: packed must be 256-byte aligned");
  int rc = check_dtype(weight_dtype);
  if (rc != B200TA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(packed);
  __nv_bfloat16* wp = reinterpret_cast<__nv_bfloat16*>(base + kTriWOff);
  float2* sc = reinterpret_cast<float2*>(base + kTriScOff);
  int* flags = reinterpret_cast<int*>(base + kTriFlagsOff);
  const size_t elem = weight_dtype == B200TA_DTYPE_F32 ? 4 : 2;
  auto rows_of = [elem](const void* w, size_t row0) -> const void* {
    return w == nullptr ? nullptr : static_cast<const char*>(w) + row0 * kC * elem;
  };
  auto vec_of = [elem](const void* v, size_t i0) -> const void* {
    return v == nullptr ? nullptr : static_cast<const char*>(v) + i0 * elem;
  };
  constexpr int H = kTriHidden;
  // gate rows are halved: sigmoid(g) = 0.5 * tanh(g / 2) + 0.5
  for (int half = 0; half < 2; ++half) {  // a channels, then b channels
    fold_rows_kernel<<<H, kC, 0, s>>>(rows_of(w_g_in, half * H), H, nullptr, 0, vec_of(b_g_in, half * H), ln_in_w, ln_in_b,
                                      weight_dtype, 0, H, 0.5f, wp + size_t(half * 2 * H) * kC, sc + half * 2 * H, flags);
    fold_rows_kernel<<<H, kC, 0, s>>>(rows_of(w_p_in, half * H), H, nullptr, 0, vec_of(b_p_in, half * H), ln_in_w, ln_in_b,
                                      weight_dtype, 0, 0, 1.f, wp + size_t(half * 2 * H + H) * kC, sc + half * 2 * H + H,
                                      flags);
  }
  fold_rows_kernel<<<kC, kC, 0, s>>>(w_g_out, kC, nullptr, 0, b_g_out, ln_in_w, ln_in_b, weight_dtype, 0, kC, 0.5f,
                                     wp + size_t(kTriInRows) * kC, sc + kTriInRows, flags);
  fold_rows_kernel<<<kC, kC, 0, s>>>(w_p_out, kC, nullptr, 0, b_p_out, ln_out_w, ln_out_b, weight_dtype, 0, 0, 1.f,
                                     wp + size_t(kTriInRows + kC) * kC, sc + kTriInRows + kC, flags);
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

int b200ta_pack_transition_weights(const void* ln_w, const void* ln_b, const void* w1, const void* w2,
                                   int weight_dtype, void* packed, void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(w1 && w2 && packed, "pack_transition_weights: NULL pointer");
  B200TA_REQUIRE((ln_w == nullptr) == (ln_b == nullptr), "pack_transition_weights: pass both LayerNorm vectors or neither");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "pack_transition_weights: packed must be 256-byte aligned");
  int rc = check_dtype(weight_dtype);
  if (rc != B200TA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(packed);
  // gate rows are halved: silu(g) = h + h * tanh(h) with h = g / 2
  // (the LayerNorm is not folded into these rows: the kernel normalises the rows of x as the eager module does)
  fold_rows_kernel<<<kTransRows, kC, 0, s>>>(w1, kTransRows, nullptr, 0, nullptr, nullptr, nullptr, weight_dtype,
                                             kHidden, kTransRows, 0.5f,
                                             reinterpret_cast<__nv_bfloat16*>(base + kTransW1Off),
                                             reinterpret_cast<float2*>(base + kTransScOff),
                                             reinterpret_cast<int*>(base + kTransFlagsOff));
  pack_transition_layernorm(ln_w, ln_b, weight_dtype, base, s);
  convert_kernel<<<(kC * kHidden + 255) / 256, 256, 0, s>>>(w2, weight_dtype, size_t(kC) * kHidden,
                                                            reinterpret_cast<__nv_bfloat16*>(base + kTransW2Off), nullptr);
  convert_kernel<<<1, kC, 0, s>>>(nullptr, weight_dtype, kC, nullptr, reinterpret_cast<float*>(base + kTransB2Off));
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

int b200ta_pack_relu_transition_weights(const void* ln_w, const void* ln_b, const void* w1, const void* b1,
                                        const void* w2, const void* b2, int weight_dtype, void* packed,
                                        void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(w1 && w2 && packed, "pack_relu_transition_weights: NULL pointer");
  B200TA_REQUIRE((ln_w == nullptr) == (ln_b == nullptr), "pack_relu_transition_weights: pass both LayerNorm vectors or neither");
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(packed) & 255u) == 0, "pack_relu_transition_weights: packed must be 256-byte aligned");
  int rc = check_dtype(weight_dtype);
  if (rc != B200TA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  char* base = static_cast<char*>(packed);
  // the 512 hidden rows (with the first linear's bias in their constant term) take the value half; the gate half
  // is zero and unused by the ReLU form of the kernel
  fold_rows_kernel<<<kTransRows, kC, 0, s>>>(w1, kHidden, nullptr, 0, b1, nullptr, nullptr, weight_dtype, 0, 0, 1.f,
                                             reinterpret_cast<__nv_bfloat16*>(base + kTransW1Off),
                                             reinterpret_cast<float2*>(base + kTransScOff),
                                             reinterpret_cast<int*>(base + kTransFlagsOff));
  pack_transition_layernorm(ln_w, ln_b, weight_dtype, base, s);
  convert_kernel<<<(kC * kHidden + 255) / 256, 256, 0, s>>>(w2, weight_dtype, size_t(kC) * kHidden,
                                                            reinterpret_cast<__nv_bfloat16*>(base + kTransW2Off), nullptr);
  convert_kernel<<<1, kC, 0, s>>>(b2, weight_dtype, kC, nullptr, reinterpret_cast<float*>(base + kTransB2Off));
  B200TA_CHECK_CUDA(cudaGetLastError());
  return B200TA_OK;
}

}  // extern "C"
