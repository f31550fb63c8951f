// Tile bytecode for the sm_100a vector interpreter (shared by the host compiler and the device VM).
//
// Execution model.  A launch walks an iteration space of `num_groups` groups, each holding
// `group_elems` elements.  A reduce-free graph is one group spanning the whole (coalesced) domain and its
// chunks are dealt round-robin to the CTAs ("flat" mode).  A graph with reductions makes one group per
// kept (non-reduced) coordinate; a CTA, or a power-of-two slice of a warp, owns a group and loops over
// its chunks ("group" mode).  A chunk is one or more rounds of up to `16 * tg` consecutive elements of a group: in a
// round thread `t` of the group owns four 4-element granules at `4*t + g*4*tg` (g = 0..3), so every global access
// is a coalesced 16-byte (fp32), 8-byte (fp16/bf16) or 4-byte (bool) vector.  Chunks of several rounds spread the
// per-chunk work (barrier waits, bookkeeping, for single-micro-op bodies also the dispatch) over more elements.
//
// The machine is an accumulator machine.  The 16-lane accumulator is the only vector state in registers;
// every other operand is read where it already lives: an input tensor's chunk in the shared-memory ring
// that a producer warp fills with bulk async copies (cp.async.bulk + mbarrier), a thread-private
// shared-memory temporary, a scalar register, or an immediate.  The scalar side (accumulator + 12 named
// scalars) holds values that are constant inside a group (reduce results, per-channel parameters).  The
// program is cut into sections
// PRO_0, BODY_0, PRO_1, BODY_1, ... : PRO_p runs once per group on the scalar side (it finalises the
// reductions accumulated by BODY_{p-1}); BODY_p runs once per chunk on the vector side.
//
// This plays the role of the reference's instruction set header (src/isa.h:59-228 opcodes,
// src/isa.h:261-299 instruction head, src/isa.h:2388-2451 entry word); the encoding is new.
#ifndef DVM_B200_ISA_H_
#define DVM_B200_ISA_H_

#include <cstdint>

namespace dvmb {

constexpr int kMaxTensors = 16;
constexpr int kMaxCodeWords = 288;   // words of the program a launch carries (scalar sections + micro-ops)
constexpr int kMaxKept = 3;
constexpr int kMaxEnum = 4;
constexpr int kNumTemps = 6;            // thread-private 8-lane temporaries in shared memory
constexpr int kNumSRegs = 12;
constexpr int kNumRSlots = 4;
constexpr int kMaxPhases = 4;        // BODY sections
constexpr int kLanes = 16;           // elements per thread per vector register (four 4-element granules)
constexpr int kAccIdx = 15;          // `dst` value meaning "the accumulator"

// Element types as stored in global memory (same numbering as dvm::DataType).
enum : uint32_t { T_BOOL = 0, T_F16 = 1, T_BF16 = 2, T_F32 = 3, T_I32 = 4, T_I64 = 5 };

enum Opcode : uint32_t {
  OP_END = 0,
  OP_LD,     // unused (inputs are operands of kind K_TENSOR)
  OP_ST,     // tensor[sub] <- acc
  OP_COPY,   // acc <- operand
  OP_MOV,    // temp[dst] <- acc (vector side) / sreg[dst] <- sacc (scalar side)
  OP_UN,     // acc <- unary[sub](acc)
  OP_BIN,    // acc <- binary[sub](acc, operand)
  OP_CMP,    // acc <- cmp[sub](acc, operand) ? 1 : 0   (in the operand representation)
  OP_SEL,    // acc <- acc != 0 ? operand : operand2
  OP_CVT,    // acc <- convert[sub](acc)
  OP_RACC,   // partial[sub&3] (op)= lanes of acc        (vector side only)
  OP_RFIN,   // sacc <- reduce over the group of partial[sub&3]; partial reset   (scalar side only)
  OP_RINIT,  // partial[sub&3] <- identity
  OP_COUNT
};

// Scalar sections of a lowered program: the host replaces the opcode byte of the common forms (no rounding, operand an
// immediate, a scalar register or the accumulator) by one of these flat handler ids, so that the device dispatches once
// per word; every other word keeps its opcode (< SOP_FIRST) and takes the general decode path.
enum ScalarOp : uint32_t {
  SOP_FIRST = 16,
  SOP_COPY = SOP_FIRST, SOP_MOV, SOP_RINIT, SOP_RFIN,
  SOP_UN_FIRST,                      // + UnKind
  SOP_BIN_FIRST = SOP_UN_FIRST + 12, // + BinKind
  SOP_CVT_FIRST = SOP_BIN_FIRST + 17,   // + CvtKind (V_F2I .. V_NEZ_I)
  SOP_MOV_END = SOP_CVT_FIRST + 4,   // SOP_MOV / SOP_RINIT as the last word of a section: the section ends inside the
  SOP_RINIT_END,                     // handler (no END word follows, which saves its dispatch)
  SOP_RSTD_FAST,                     // sacc <- 1 / sqrt(sacc * imm + imm'), fast division: the four words Mul #imm, Add #imm',
                                     // Sqrt, RDivFast #1.0 as one; imm' is read from the following word, which is skipped
  SOP_RFIN2,                         // two sum reductions finished behind one CTA barrier: partial (sub & 3) -> scalar register dst,
                                     // partial (sub >> 2 & 3) -> scalar register oidx and sacc (the words RFIN, MOV, RFIN, MOV as one;
                                     // each sum is combined in the order of a single RFIN)
  SOP_COUNT
};

enum UnKind : uint32_t { U_SQRT = 0, U_ABS, U_LOG, U_EXP, U_ROUND, U_FLOOR, U_CEIL, U_TRUNC, U_ISFINITE, U_ABS_I,
                         U_EXP_FAST,   // exp through ex2.approx (relative error about 1e-6): values that never reach an exact-class op
                         U_NOP };
static_assert(U_NOP + 1 == 12, "ScalarOp numbering follows UnKind");

enum BinKind : uint32_t {
  B_ADD = 0, B_SUB, B_MUL, B_DIV, B_MAX, B_MIN, B_POW, B_RSUB, B_RDIV,
  B_ADD_I, B_SUB_I, B_MUL_I, B_MAX_I, B_MIN_I, B_RSUB_I,
  B_DIV_FAST, B_RDIV_FAST,   // 2-ulp full-range division, same eligibility rule as U_EXP_FAST
  B_COUNT
};
static_assert(B_COUNT == 17, "ScalarOp numbering follows BinKind");

enum CmpKind : uint32_t { C_EQ = 0, C_NE, C_GT, C_GE, C_LT, C_LE };

enum CvtKind : uint32_t {
  V_F2I = 0,   // float -> int32, truncation toward zero (C cast semantics)
  V_I2F,       // int32 -> float
  V_NEZ_F,     // float != 0 -> int 0/1
  V_NEZ_I,     // int   != 0 -> int 0/1
  V_RND        // no arithmetic: only the rounding field applies (fp32 -> fp16/bf16 precision)
};

enum RedKind : uint32_t { R_SUM = 0, R_MAX, R_MIN };

// K_TENSOR: chunk of input tensor `idx`, converted to the 32-bit register form on read.
// K_TEMP: thread-private temporary `idx`.
enum OperandKind : uint32_t { K_TENSOR = 0, K_SREG = 1, K_IMM = 2, K_ACC = 3, K_TEMP = 4 };

enum Rounding : uint32_t { RN_NONE = 0, RN_F16 = 1, RN_BF16 = 2 };

// Instruction word (64 bit):
//   [31:0] imm32  [39:32] opcode  [47:40] sub  [51:48] operand kind  [55:52] operand index
//   [59:56] dst   [61:60] rounding  [62] integer representation flag  [63] scalar-side flag
// OP_SEL packs its second operand into sub: kind in sub[7:4], index in sub[3:0] (never an immediate).
struct Insn {
  static constexpr uint64_t make(uint32_t opc, uint32_t sub, uint32_t okind, uint32_t oidx, uint32_t dst,
                                 uint32_t rnd, uint32_t isint, uint32_t scalar, uint32_t imm) {
    return (uint64_t)imm | ((uint64_t)(opc & 0xff) << 32) | ((uint64_t)(sub & 0xff) << 40) |
           ((uint64_t)(okind & 0xf) << 48) | ((uint64_t)(oidx & 0xf) << 52) | ((uint64_t)(dst & 0xf) << 56) |
           ((uint64_t)(rnd & 0x3) << 60) | ((uint64_t)(isint & 1) << 62) | ((uint64_t)(scalar & 1) << 63);
  }
};

#define DVMB_IMM(w) ((uint32_t)(w))
#define DVMB_OPC(w) ((uint32_t)((w) >> 32) & 0xffu)
#define DVMB_SUB(w) ((uint32_t)((w) >> 40) & 0xffu)
#define DVMB_OKIND(w) ((uint32_t)((w) >> 48) & 0xfu)
#define DVMB_OIDX(w) ((uint32_t)((w) >> 52) & 0xfu)
#define DVMB_DST(w) ((uint32_t)((w) >> 56) & 0xfu)
#define DVMB_RND(w) ((uint32_t)((w) >> 60) & 0x3u)
#define DVMB_ISINT(w) ((uint32_t)((w) >> 62) & 0x1u)
#define DVMB_SCALAR(w) ((uint32_t)((w) >> 63) & 0x1u)

// ---- micro-ops ------------------------------------------------------------------------------------
// BODY sections are not executed from the instruction words above but from micro-ops the host lowers them
// to once the tensor addresses are known: one flat, dense handler id per word, every parameter resolved
// (ring offset, register index, immediate), no tensor-descriptor reads on the fast paths.
//   [7:0] handler   [15:8] aux   [31:16] arg16   [63:32] imm32
enum UopHandler : uint32_t {
  UH_END = 0,
  // operand fetches; aux[1:0] = destination (UD_B / UD_ACC), aux[5:2] = tensor slot
  UH_LDR_F32, UH_LDR_F16, UH_LDR_BF16, UH_LDR_U8,   // from the ring stage into b, arg16 = ring offset / 16
  UH_LDRA_F32, UH_LDRA_F16, UH_LDRA_BF16, UH_LDRA_U8,   // the same into acc (one handler per destination: no test on the way)
  UH_LDG,                                           // from global memory through the tensor descriptor
  UH_LDT,                                           // thread-private temporary arg16
  UH_LDS,                                           // scalar register arg16, splat
  UH_LDI,                                           // imm32, splat
  UH_MOVA,                                          // destination <- acc
  UH_SQR,                                           // acc <- acc * acc (a product whose operand is the accumulator itself)
  UH_RCP,                                           // acc <- 1 / acc, 1 ulp (the fast form of an immediate 1.0 divided by acc)
  UH_STT,                                           // temporary arg16 <- acc
  // acc <- op(acc, b)
  UH_BINV_FIRST,
  UH_BINV_LAST = UH_BINV_FIRST + B_COUNT - 1,
  // acc <- op(acc, imm32)
  UH_BINS_FIRST,
  UH_BINS_LAST = UH_BINS_FIRST + B_COUNT - 1,
  // acc <- op(acc, scalar register arg16)
  UH_BINR_FIRST,
  UH_BINR_LAST = UH_BINR_FIRST + B_COUNT - 1,
  UH_UN_FIRST,
  UH_UN_LAST = UH_UN_FIRST + U_NOP,
  UH_RND_F16, UH_RND_BF16,
  // compares: aux[2:0] = CmpKind; the _S forms take UA_CMP_SREG = scalar register arg16, else imm32
  UH_CMP_F_V, UH_CMP_F_S, UH_CMP_I_V, UH_CMP_I_S,
  UH_PRED_F, UH_PRED_I,                             // lane mask <- acc != 0
  UH_SELM,                                          // acc <- lane mask ? acc : b
  UH_CVT_F2I, UH_CVT_I2F, UH_CVT_NEZ_F, UH_CVT_NEZ_I,
  UH_RACC_SUM, UH_RACC_MAX, UH_RACC_MIN,            // arg16 = partial slot; any chunk (lanes past the end are masked)
  UH_RACCF_FIRST,                                   // full chunks: handler = first + kind * 4 + partial slot
  UH_RACCF_LAST = UH_RACCF_FIRST + 11,
  UH_ST_F32, UH_ST_F16, UH_ST_BF16, UH_ST_U8,       // dense, aligned tensor arg16: vector stores
  UH_STG,                                           // any tensor arg16
  // ---- fused forms (full chunks only): the host's peephole pass replaces frequent neighbours by one handler, so that
  // the pair costs one dispatch; each computes exactly what its parts compute, in the same order and rounding
  UH_LDOP_FIRST,                                    // b <- ring operand; acc <- acc (add | sub | mul) b:
  UH_LDOP_LAST = UH_LDOP_FIRST + 8,                 //   handler = first + FusedOp * 3 + FusedType, arg16 = ring offset / 16
  UH_LDSUM_FIRST,                                   // acc <- ring operand; partial 0 += lanes of acc: first + FusedType
  UH_LDSUM_LAST = UH_LDSUM_FIRST + 2,
  UH_LDSUBR_FIRST,                                  // acc <- ring operand - scalar register imm32: first + FusedType
  UH_LDSUBR_LAST = UH_LDSUBR_FIRST + 2,
  UH_SQRSUM0, UH_SQRSUM1,                           // acc <- acc * acc; partial 0 / 1 += lanes of acc
  UH_SUBR_MULR, UH_MULR_ADDR, UH_MULR_MULR,         // two scalar-register operands: arg16 = first | second << 8
  UH_SIGMOID_FAST,                                  // acc <- 1 / (1 + exp(-acc)) in the fast forms (mul -1, EXP_FAST, add 1, RCP)
  UH_LD2OP_FIRST,                                   // acc <- ring operand arg16; b <- ring operand imm32 (same type); acc <- acc
  UH_LD2OP_LAST = UH_LD2OP_FIRST + 8,               //   (add | sub | mul) b: first + FusedOp * 3 + FusedType
  UH_MULR_MULR_ADDR,                                // three scalar registers: arg16 = first | second << 4 | third << 8
  // the two passes of a normalisation over a ring operand x (arg16 = ring offset / 16, scalar registers in imm32, four
  // bits each): the sum of (x - s0)^2 into partial 0 / 1, and ((x - s0) * s1) * s2 + s3
  UH_LDVAR_FIRST,                                   // first + slot * 3 + FusedType
  UH_LDVAR_LAST = UH_LDVAR_FIRST + 5,
  UH_LDNORM_FIRST,                                  // first + FusedType
  UH_LDNORM_LAST = UH_LDNORM_FIRST + 2,
  UH_LDSIGM_FIRST,                                  // acc <- fast sigmoid of ring operand arg16: first + FusedType
  UH_LDSIGM_LAST = UH_LDSIGM_FIRST + 2,
  UH_LDMUL2_FIRST,                                  // acc <- (acc * ring operand arg16) * ring operand imm32 (one type; b keeps
  UH_LDMUL2_LAST = UH_LDMUL2_FIRST + 2,             //   the second): first + FusedType
  // a whole normalisation body: ((x - s0) * s1) * s2 + s3 over ring operand x (arg16 = ring offset / 16; imm32 = the four
  // scalar registers, four bits each, and the result tensor's slot in bits 16-19), stored as a vector of the operand's
  // own type; with UA_LOOP the handler runs every remaining full round of the chunk
  UH_LDNORMST_FIRST,                                // first + FusedType
  UH_LDNORMST_LAST = UH_LDNORMST_FIRST + 2,
  // the pieces of a residual RMSNorm + gated-activation graph, one dispatch each.  Ring offsets / 16 are 12 bits wide here.
  //   sum of squares of a sum:  acc <- (ring A + ring B)^2; partial 0 / 1 += lanes.  arg16 = A, imm32 = B
  UH_LD2ADDSQRSUM_FIRST,                            // first + slot * 3 + FusedType
  UH_LD2ADDSQRSUM_LAST = UH_LD2ADDSQRSUM_FIRST + 5,
  //   scaled sum times a weight, stored:  ((ring A + ring B) * sreg) * ring W -> vector store in the operands' type.
  //   arg16 = A, imm32 = B | W << 12 | result slot << 24 | sreg << 28
  UH_LD2ADDMULRMULST_FIRST,                         // first + FusedType
  UH_LD2ADDMULRMULST_LAST = UH_LD2ADDMULRMULST_FIRST + 2,
  //   gated activation, stored:  (sigmoid(ring G) * ring X) * ring Y -> vector store (fast sigmoid forms).
  //   arg16 = G, imm32 = X | Y << 12 | result slot << 24
  UH_LDSIGMMUL2ST_FIRST,                            // first + FusedType
  UH_LDSIGMMUL2ST_LAST = UH_LDSIGMMUL2ST_FIRST + 2,
  // first pass of a normalisation that needs no second one: d = x - s over ring operand x (arg16 = ring offset / 16,
  // imm32 = the scalar register of s), partial 0 += lanes of d, partial 1 += lanes of d * d; loops like the other
  // load + reduce forms
  UH_LDSTATS_FIRST,                                 // first + FusedType
  UH_LDSTATS_LAST = UH_LDSTATS_FIRST + 2,
  UH_COUNT
};
enum FusedOp : uint32_t { FO_ADD = 0, FO_SUB = 1, FO_MUL = 2 };
enum FusedType : uint32_t { FT_F32 = 0, FT_F16 = 1, FT_BF16 = 2 };   // the order of UH_LDR_F32 .. UH_LDR_BF16
static_assert(UH_COUNT <= 256, "handler ids are one byte");
enum UopDest : uint32_t { UD_B = 0, UD_ACC = 1 };
enum UopAux : uint32_t {
  UA_CMP_SREG = 0x08,  // scalar compares: the scalar is register arg16, else imm32
  UA_LOOP = 0x40,      // load + reduce and load + normalise + store forms that are a body's only micro-op: the handler runs all
                       // remaining full rounds of the chunk
  UA_LAST = 0x80       // vector stores and full-chunk reduce accumulations (plain or fused): the body ends here (no UH_END
                       // word follows, which saves its dispatch)
};

constexpr uint64_t MakeUop(uint32_t handler, uint32_t aux, uint32_t arg16, uint32_t imm) {
  return (uint64_t)(handler & 0xff) | ((uint64_t)(aux & 0xff) << 8) | ((uint64_t)(arg16 & 0xffff) << 16) |
         ((uint64_t)imm << 32);
}
#define DVMB_UH(u) ((uint32_t)(u) & 0xffu)
#define DVMB_UAUX(u) (((uint32_t)(u) >> 8) & 0xffu)
#define DVMB_UARG(u) ((uint32_t)(u) >> 16)
#define DVMB_UIMM(u) ((uint32_t)((u) >> 32))

// How a tensor's element offset is derived from (group, element-in-group).
enum AddrMode : uint32_t {
  AM_DENSE = 0,    // offset = kept part + element index (contiguous over the enumerated axes)
  AM_GRANULE = 1,  // innermost enumerated size % 4 == 0: one coordinate split per 4-element granule
  AM_ELEMENT = 2,  // coordinate split per element
  AM_SCALAR = 3    // constant inside a group (all enumerated strides are 0)
};

struct TensorDesc {
  uint64_t ptr;                // device address (the relocation site; see code.h:56-76 in the reference)
  uint32_t kstride[kMaxKept];  // element strides along the kept axes (outer -> inner)
  uint32_t estride[kMaxEnum];  // element strides along the enumerated axes, right-aligned (index 3 = innermost)
  uint8_t dtype;
  uint8_t mode;
  uint8_t vec_ok;              // granules are contiguous and aligned to 4 elements
  uint8_t layout_vec;          // the layout permits vector access (vec_ok = layout_vec && aligned address)
  uint32_t ring_off;           // byte offset of this tensor's chunk inside a ring stage, or kNoRing
  uint8_t ring_layout;         // the layout permits bulk staging (ring_off is set when the address is aligned)
  uint8_t chunk_contig;        // every chunk is one contiguous run of this tensor (its start follows from the chunk's coordinates)
  uint8_t pad[2];
};
constexpr uint32_t kNoRing = 0xffffffffu;
// Element offsets are 32-bit: a tensor bound to the vector interpreter holds fewer than 2^31 elements.

enum VmMode : uint32_t { VM_FLAT = 0, VM_GROUP = 1 };

struct VmParam {
  uint32_t mode;
  uint32_t num_groups;
  uint32_t group_elems;
  uint32_t tg;               // threads cooperating on one group
  uint32_t groups_per_cta;   // groups a CTA works on at a time
  uint32_t tcons;            // consumer threads of the CTA: tg * groups_per_cta rounded up to a multiple of 32
  uint32_t chunks;           // chunks per group
  uint32_t chunk_elems;      // elements per chunk = rounds * round_elems
  uint32_t rounds;           // a chunk is this many rounds, back to back in its ring stage: the unit the producer stages and
                             // the consumers wait for is the chunk, the unit a body's micro-ops work on is the round
  uint32_t round_elems;      // elements per round (<= 16 * tg; threads past the end idle); every round is one contiguous run
                             // of each staged tensor
  uint32_t stages_off;       // byte offset of the first ring stage in shared memory (behind the program copy)
  uint32_t stage_bytes;      // bytes of one ring stage (0: no bulk staging in this launch)
  uint32_t num_stages;
  // resident groups: every chunk of a group keeps its own ring slot from the first phase to the last, so the
  // group is read from global memory once; `cluster` CTAs share a group (cpc chunks each) and combine their
  // reductions through distributed shared memory; `sets` slot sets let the next group load behind the current one
  uint32_t resident, cluster, cpc, sets;
  uint32_t body_ring_mask[kMaxPhases];  // per BODY section: tensor slots the producer stages
  uint32_t num_temps;        // shared-memory temporaries in use
  uint32_t num_sregs;        // scalar registers in use
  uint32_t kept_size[kMaxKept];
  uint32_t enum_size[kMaxEnum];   // right-aligned, unused outer slots are 1
  uint32_t need_coords;      // some tensor uses AM_GRANULE or is staged per segment
  uint32_t body_coords_mask; // BODY sections whose vector stores address a strided tensor through the chunk coordinates
  uint32_t num_body;         // number of BODY sections
  uint32_t pro_skip_mask;    // PRO sections that hold nothing but their END word (not entered at all)
  // word offset of PRO_0, BODY_0, PRO_1, ..., PRO_n in code[]: PRO sections hold instruction words ending
  // with OP_END, BODY sections hold micro-ops ending with UH_END
  uint16_t sec[2 * kMaxPhases + 2];
  // BODY sections come twice: the one in sec[] assumes a chunk in which every lane of every thread is valid
  // (ring loads, vector stores, unmasked reductions), this one takes any chunk
  uint16_t sec_any[kMaxPhases];
  uint32_t n_tensors;
  uint32_t n_code;
  TensorDesc tensor[kMaxTensors];
  uint64_t code[kMaxCodeWords];
};

static_assert(sizeof(VmParam) <= 4096, "VmParam must fit the 4 KB kernel parameter space");

}  // namespace dvmb

#endif  // DVM_B200_ISA_H_
