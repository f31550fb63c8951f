// Host-callable entry points of the tensor-core kernels (MatMul with fused post-ops, fused attention).
#ifndef DVM_B200_MM_LAUNCH_H_
#define DVM_B200_MM_LAUNCH_H_

#include <cstdint>

#include "isa.h"

namespace dvmb {

constexpr int kMmMaxEpilogueWords = 96;
constexpr int kMmMaxEpiTensors = 8;

// A tensor the post-fusion program reads or writes, addressed by (batch0, batch1, row, column) of the
// MatMul result.  A stride of 0 broadcasts along that coordinate.
struct EpiTensor {
  uint64_t ptr;
  int64_t sb0, sb1;   // element strides along the two batch coordinates
  int64_t sm;         // element stride along rows
  int32_t sn;         // element stride along columns (0 or 1 for the vector paths)
  uint32_t dtype;
};

// One batched MatMul  C[b0,b1] = op(A[..]) * op(B[..]) (+ bias), rounded to the operand type, followed by the
// fused post-ops.  Batch coordinates: b = b0 * batch1 + b1; an operand's batch slice is
// z = b0 * mul0 + b1 * mul1 (multipliers 0 broadcast the operand).
struct MmParam {
  uint32_t M, N, K;
  uint32_t batch0, batch1;
  uint32_t a_mmajor;        // 1: A is stored [K, M] (trans_a), 0: A is stored [M, K]
  uint32_t b_kmajor;        // 1: B is stored [N, K] (trans_b), 0: B is stored [K, N]
  uint32_t in_dtype;        // T_F16 or T_BF16: operand type and the type the product is rounded to
  uint32_t bias_dtype;      // element type of bias (ignored when bias_ptr == 0)
  uint32_t a_mul0, a_mul1, a_batches;   // batch-slice multipliers and slice count of A
  uint32_t b_mul0, b_mul1, b_batches;
  uint64_t a_ptr, b_ptr, bias_ptr;
  // post-fusion program: instruction words (isa.h Insn) over 16 consecutive columns of one row, ending with
  // OP_END; operand kind K_TENSOR with index `mma_slot` names the rounded product itself
  uint32_t n_tensors;
  uint32_t mma_slot;
  uint32_t num_temps;
  uint32_t group_m;         // row blocks swept together over all column blocks (L2 reuse of the A panel); set by the launcher
  uint32_t fast_store_slot; // set by the launcher: the post-fusion program is just "store the product to tensor <slot>" (in the
                            // operand type or widened to fp32), which the kernel does without interpreting; 0xffffffff otherwise
  // set by the launcher: the post-fusion program is the gated form  y = x / (c2 + exp(c1 * (x + c0 * x^3)))  of the
  // rounded product x (tanh-GeLU written through the exponential, c0 = 0.044715, c1 = -2 sqrt(2/pi), c2 = 1), rounded to
  // the operand type and stored to tensor <gate_slot>: the kernel computes it in registers with the interpreter's own
  // operations in the interpreter's order (same bits) instead of interpreting eleven words per strip; 0xffffffff otherwise
  uint32_t gate_slot;
  uint32_t gate_c[3];
  uint32_t leave_sms;       // set by the planner: SMs this launch leaves free (a collective runs beside it); 0 = none
  EpiTensor tensor[kMmMaxEpiTensors];
  uint64_t epilogue[kMmMaxEpilogueWords];
};

// Enqueue the MatMul.  Returns 0, a cudaError_t (> 0), or a negative code for an unsupported shape.
int LaunchMatMul(const MmParam &p, void *stream);
// True when the tcgen05 path can take this problem (TMA alignment rules); otherwise LaunchMatMul runs the
// general SIMT kernel.
bool MatMulUsesTensorCores(const MmParam &p);
unsigned int ReadMatMulStatus();

// Fused attention  O[b,h] = softmax(scale * Q[b,h] K[b,h]^T) V[b,h]  (non-causal), bf16 or fp16 operands,
// fp32 softmax, result in the operand type.  Q [B0,B1,Sq,D], K and V [B0,B1,Skv,D], all contiguous.
struct AttnParam {
  uint32_t batch;           // B0 * B1
  uint32_t sq, skv, d;      // d is 64 or 128
  uint32_t dtype;           // T_F16 or T_BF16
  uint32_t scale_bits;      // scale in the operand type's register form (fp32 bits)
  uint32_t scale_first;     // 1: the score is rounded to the operand type, scaled, rounded again (the graph's order)
  uint32_t pad0;
  uint64_t q_ptr, k_ptr, v_ptr, o_ptr;
};
int LaunchAttention(const AttnParam &p, void *stream);
bool AttentionSupported(const AttnParam &p);
unsigned int ReadAttentionStatus();

}  // namespace dvmb

#endif  // DVM_B200_MM_LAUNCH_H_
