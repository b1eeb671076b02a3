// One call for a whole triangle-attention node: prologue -> attention -> epilogue on one stream, with the
// intermediates (q/k/v/gate planes, triangle bias, gated attention output) in a caller-provided workspace.
#include <mutex>

#include "common.cuh"
#include "layout.h"

namespace b200ta {
namespace {

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct NodeWorkspace {
  size_t qkvg_off, bias_off, og_off, total;
  int s_pad;
};

NodeWorkspace plan_workspace(int B, int N) {
  NodeWorkspace w;
  const size_t positions = size_t(B) * N * N;
  w.s_pad = (N + 7) / 8 * 8;
  w.qkvg_off = 0;
  w.bias_off = align_up(positions * 4 * kHeads * kHeadDim * 2);
  w.og_off = w.bias_off + align_up(size_t(B) * kHeads * N * w.s_pad * 2);
  w.total = w.og_off + align_up(positions * kC * 2);
  return w;
}

}  // namespace

// Shared by b200ta_node_forward and the static-scratch variant.
int node_forward_impl(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed, float eps,
                      const int32_t* lengths, int64_t ls_b, int64_t ls_r, int empty_row_mode, int add_residual,
                      void* out, int64_t os_b, int64_t os_r, int64_t os_s, void* workspace, size_t workspace_bytes,
                      int B, int N, void* stream) {
  B200TA_REQUIRE(z && packed && out && workspace, "node_forward: NULL pointer");
  B200TA_REQUIRE(B > 0 && N > 0, "node_forward: bad sizes B=%d N=%d", B, N);
  B200TA_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) == 0, "node_forward: workspace must be 256-byte aligned");
  const NodeWorkspace w = plan_workspace(B, N);
  B200TA_REQUIRE(workspace_bytes >= w.total, "node_forward: workspace of %zu bytes is smaller than the %zu needed",
                 workspace_bytes, w.total);
  char* ws = static_cast<char*>(workspace);
  void* qkvg = ws + w.qkvg_off;
  void* bias = ws + w.bias_off;
  void* og = ws + w.og_off;
  const int64_t S = N, R = N;
  // q/k/v/g planes [4][B*R][H][S][D]
  const int64_t qs_s = kHeadDim, qs_h = S * kHeadDim, qs_br = kHeads * qs_h, qs_which = int64_t(B) * R * qs_br;
  // bias [B][H][S][S_pad]
  const int64_t bs_q = w.s_pad, bs_h = S * bs_q, bs_b = kHeads * bs_h;
  int rc = b200ta_prologue(z, zs_b, zs_r, zs_s, packed, eps, qkvg, qs_which, qs_br, qs_h, qs_s, 1, bias, bs_b, bs_h,
                           bs_q, 1, B, int(R), int(S), w.s_pad, stream);
  if (rc != B200TA_OK) return rc;
  const __nv_bfloat16* planes = static_cast<const __nv_bfloat16*>(qkvg);
  // og [B*R][S][H][D]
  rc = b200ta_attention(planes, planes + qs_which, planes + 2 * qs_which, planes + 3 * qs_which, qs_br, qs_h, qs_s, bias,
                        bs_b, bs_h, bs_q, lengths, ls_b, ls_r, og, S * kC, kC, kHeadDim, nullptr,
                        0.17677669529663687f /* 1/sqrt(32) */, empty_row_mode, B, int(R), int(S), w.s_pad, stream);
  if (rc != B200TA_OK) return rc;
  return b200ta_epilogue(og, R * S * kC, S * kC, kC, packed, add_residual ? z : nullptr, zs_b, zs_r, zs_s, out, os_b, os_r,
                         os_s, B, int(R), int(S), stream);
}

}  // namespace b200ta

extern "C" {

size_t b200ta_node_workspace_bytes(int B, int N) {
  if (B <= 0 || N <= 0) return 0;
  return b200ta::plan_workspace(B, N).total;
}

int b200ta_node_forward(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed, float eps,
                        const int32_t* lengths, int64_t ls_b, int64_t ls_r, int empty_row_mode, int add_residual,
                        void* out, int64_t os_b, int64_t os_r, int64_t os_s, void* workspace, size_t workspace_bytes,
                        int B, int N, void* stream) {
  return b200ta::node_forward_impl(z, zs_b, zs_r, zs_s, packed, eps, lengths, ls_b, ls_r, empty_row_mode, add_residual,
                                   out, os_b, os_r, os_s, workspace, workspace_bytes, B, N, stream);
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------
// Allocation-free variant: the node's intermediates live in a fixed device array that is part of the library
// image, for callers that may not allocate device memory at all (see include/b200ta.h).
// ---------------------------------------------------------------------------------------------------------
namespace b200ta {
namespace {

// Largest problem the built-in scratch holds: B*N*N pair positions (for example one 64 x 64 pair tensor).
constexpr int kStaticMaxPositions = 4096;
// q/k/v/gate planes (1 KiB per position) + triangle bias (at most 256 KiB within the position limit) + gated
// attention output (256 B per position) + alignment slack: about 5.25 MiB on every device that loads the library.
constexpr size_t kStaticScratchBytes = size_t(kStaticMaxPositions) * 1024 + 262144 + size_t(kStaticMaxPositions) * 256 + 1024;

static __device__ __align__(256) unsigned char g_node_scratch[kStaticScratchBytes];

std::mutex g_scratch_mutex;
void* g_scratch_addr[64] = {};  // per device: device address of g_node_scratch

// In host code `g_node_scratch` is only a handle for the runtime, not a device address: the address a kernel
// can use has to be asked for, once per device and with that device current.
int static_scratch_address(void** out) {
  int dev = 0;
  B200TA_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200TA_ERR_INVALID, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    B200TA_CHECK_CUDA(cudaGetSymbolAddress(&ptr, g_node_scratch));
    if (ptr == nullptr) return fail(B200TA_ERR_CUDA, "cudaGetSymbolAddress returned a null scratch address");
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return B200TA_OK;
}

}  // namespace
}  // namespace b200ta

extern "C" {

int b200ta_node_static_max_positions(void) { return b200ta::kStaticMaxPositions; }

int b200ta_node_forward_static(const void* z, int64_t zs_b, int64_t zs_r, int64_t zs_s, const void* packed, float eps,
                               const int32_t* lengths, int64_t ls_b, int64_t ls_r, int empty_row_mode,
                               int add_residual, void* out, int64_t os_b, int64_t os_r, int64_t os_s, int B, int N,
                               void* stream) {
  using namespace b200ta;
  B200TA_REQUIRE(B > 0 && N > 0, "node_forward_static: bad sizes B=%d N=%d", B, N);
  const long long positions = (long long)B * N * N;
  if (positions > kStaticMaxPositions)
    return fail(B200TA_ERR_UNSUPPORTED,
                "node_forward_static: B*N*N = %lld pair positions exceed the %d the built-in scratch holds; use "
                "b200ta_node_forward with a caller-provided workspace",
                positions, kStaticMaxPositions);
  const size_t need = b200ta_node_workspace_bytes(B, N);
  if (need > kStaticScratchBytes)
    return fail(B200TA_ERR_UNSUPPORTED, "node_forward_static: needs %zu scratch bytes, the built-in array has %zu", need,
                kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc != B200TA_OK) return rc;
  // Nothing in the scratch has to start at zero: every byte a later stage reads (projections, bias including its
  // zeroed key padding, gated output) is written by an earlier stage of this same call.
  return node_forward_impl(z, zs_b, zs_r, zs_s, packed, eps, lengths, ls_b, ls_r, empty_row_mode, add_residual, out, os_b,
                           os_r, os_s, scratch, kStaticScratchBytes, B, N, stream);
}

}  // extern "C"
