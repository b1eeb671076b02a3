// Byte layout of the packed (LayerNorm-folded) weight buffers.
#pragma once
#include <stddef.h>

namespace b200ta {

constexpr int kC = 128;         // pair channels
constexpr int kHeads = 4;
constexpr int kHeadDim = 32;
constexpr int kHidden = 512;    // transition hidden width

// ---- triangle-attention node -------------------------------------------------
// Rows of the folded in-projection: q(128) k(128) v(128) g(128) bias(4) pad(12).
constexpr int kNodeRows = 528;
constexpr size_t kNodeWOff = 0;                                   // bf16 [528][128]
constexpr size_t kNodeScOff = kNodeWOff + size_t(kNodeRows) * kC * 2;  // float2 [528] {rowsum, const}
constexpr size_t kNodeWoOff = kNodeScOff + size_t(kNodeRows) * 8;      // bf16 [128][128] (o_proj)
constexpr size_t kNodeBoOff = kNodeWoOff + size_t(kC) * kC * 2;        // float [128]
constexpr size_t kNodeFlagsOff = kNodeBoOff + kC * 4;                  // int [4]: {input is layer-normalised by the kernel, 0, 0, 0}
constexpr size_t kNodePackBytes = ((kNodeFlagsOff + 16 + 255) / 256) * 256;

// ---- transition ---------------------------------------------------------------
// Rows of the first linear as bf16: value(512) then gate(512, pre-halved for the
// tanh form of silu).  The LayerNorm is applied to the rows of x by the kernel (gamma, beta at kTransLnOff),
// as the eager module does, not folded into the weights.  The ReLU form (linear_2(relu(linear_1(LN(x)))), both with biases) keeps its 512 hidden rows
// in the value half, leaves the gate half zero and adds the second linear's bias from kTransB2Off.
constexpr int kTransRows = 2 * kHidden;
constexpr size_t kTransW1Off = 0;                                         // bf16 [1024][128]
constexpr size_t kTransScOff = kTransW1Off + size_t(kTransRows) * kC * 2; // float2 [1024]: {unused, bias of the row} (ReLU form)
constexpr size_t kTransW2Off = kTransScOff + size_t(kTransRows) * 8;      // bf16 [128][512]
constexpr size_t kTransFlagsOff = kTransW2Off + size_t(kC) * kHidden * 2;   // int [4]: {LayerNorm applied by the kernel, activation: 0 SwiGLU / 1 ReLU, 0, 0}
constexpr size_t kTransB2Off = kTransFlagsOff + 16;                         // float [128]: bias of the second linear (ReLU form; zero otherwise)
constexpr size_t kTransLnOff = kTransB2Off + kC * 4;                        // float [256]: LayerNorm gamma[128] | beta[128]
constexpr size_t kTransPackBytes = ((kTransLnOff + 2 * kC * 4 + 255) / 256) * 256;

// ---- triangle multiplication ---------------------------------------------------
// Folded rows: gate a(128, pre-halved) value a(128) gate b(128, pre-halved) value b(128) of the input projections,
// then the output gate (128, pre-halved; LayerNorm = norm_in) and the output projection (128; LayerNorm = norm_out).
constexpr int kTriHidden = 128;
constexpr int kTriInRows = 4 * kTriHidden;
constexpr int kTriRows = kTriInRows + 2 * kC;
constexpr size_t kTriWOff = 0;                                       // bf16 [768][128]
constexpr size_t kTriScOff = kTriWOff + size_t(kTriRows) * kC * 2;   // float2 [768] {rowsum, const}
constexpr size_t kTriFlagsOff = kTriScOff + size_t(kTriRows) * 8;    // int [4]
constexpr size_t kTriPackBytes = ((kTriFlagsOff + 16 + 255) / 256) * 256;

}  // namespace b200ta
