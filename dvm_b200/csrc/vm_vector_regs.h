// Inline-PTX building blocks of the vector interpreter's hidden register file.
//
// The vector state of a consumer thread - accumulator va0..15, operand register vb0..15 and the
// reduction partials vp0..3 - is held in PTX registers that are declared once at the top of the kernel and
// are named only inside inline assembly.  The C++ compiler therefore carries no vector value across the
// dispatch loop (nothing to copy where the handlers' control flow merges) and ptxas keeps each register
// in place for the whole kernel.  Lane i of a register belongs to granule i / 4 of the thread (four
// consecutive elements); granule g sits 4 * tg elements after granule g - 1 inside a chunk.
#ifndef DVM_B200_VM_VECTOR_REGS_H_
#define DVM_B200_VM_VECTOR_REGS_H_

#define DV_LN(M, ...)                                                                                             \
  M(0, __VA_ARGS__) M(1, __VA_ARGS__) M(2, __VA_ARGS__) M(3, __VA_ARGS__) M(4, __VA_ARGS__) M(5, __VA_ARGS__)     \
  M(6, __VA_ARGS__) M(7, __VA_ARGS__) M(8, __VA_ARGS__) M(9, __VA_ARGS__) M(10, __VA_ARGS__) M(11, __VA_ARGS__)   \
  M(12, __VA_ARGS__) M(13, __VA_ARGS__) M(14, __VA_ARGS__) M(15, __VA_ARGS__)
// pairs (a, b) of neighbouring lanes
#define DV_PAIRS(M, ...)                                                                              \
  M("0", "1", __VA_ARGS__) M("2", "3", __VA_ARGS__) M("4", "5", __VA_ARGS__) M("6", "7", __VA_ARGS__) \
  M("8", "9", __VA_ARGS__) M("10", "11", __VA_ARGS__) M("12", "13", __VA_ARGS__) M("14", "15", __VA_ARGS__)

#define DV_DECLARE ".reg .b32 va<16>, vb<16>, vp<4>;"
// lane templates that name their register (R = "va" or "vb"): the looping handlers work on two rounds at a time, one in
// each vector register, so that the loads and the arithmetic of the two overlap
#define DV_LNR(M, R, ...)                                                                                         \
  M(0, R, __VA_ARGS__) M(1, R, __VA_ARGS__) M(2, R, __VA_ARGS__) M(3, R, __VA_ARGS__) M(4, R, __VA_ARGS__)         \
  M(5, R, __VA_ARGS__) M(6, R, __VA_ARGS__) M(7, R, __VA_ARGS__) M(8, R, __VA_ARGS__) M(9, R, __VA_ARGS__)         \
  M(10, R, __VA_ARGS__) M(11, R, __VA_ARGS__) M(12, R, __VA_ARGS__) M(13, R, __VA_ARGS__) M(14, R, __VA_ARGS__)    \
  M(15, R, __VA_ARGS__)
#define DV_SUBS_LANE_R(i, R, X) "sub.rn.f32 " R #i ", " R #i ", %0;\n\t"
#define DV_SQRRN_LANE_R(i, R, X) "mul.rn.f32 " R #i ", " R #i ", " R #i ";\n\t"
#define DV_CSQR_LANE_R(i, R, X) "sub.rn.f32 " R #i ", " R #i ", %0;\n\tmul.rn.f32 " R #i ", " R #i ", " R #i ";\n\t"
// ((x - %0) * %1) * %2 + %3 on two neighbouring lanes at a time: the subtraction and the two multiplications as packed
// f32x2 operations (%0..%2 hold the scalar twice, as a 64-bit pair), the addition per lane - a packed addition behind a
// packed multiplication is contracted into a fused multiply-add by the assembler, which would change the result (so is
// a packed fused multiply-add by one in its place; a packed addition under an always-true predicate keeps its rounding
// but measured slower than the two additions per lane)
#define DV_NORM2_PAIR_R(a, b, R, D)                                                                              \
  "mov.b64 " D ", {" R a ", " R b "};\n\tsub.rn.f32x2 " D ", " D ", %0;\n\tmul.rn.f32x2 " D ", " D ", %1;\n\t"        \
  "mul.rn.f32x2 " D ", " D ", %2;\n\tmov.b64 {" R a ", " R b "}, " D ";\n\t"                                         \
  "add.rn.f32 " R a ", " R a ", %3;\n\tadd.rn.f32 " R b ", " R b ", %3;\n\t"
#define DV_NORM2_R(R)                                                                                            \
  "{\n\t.reg .b64 d<8>;\n\t" DV_NORM2_PAIR_R("0", "1", R, "d0") DV_NORM2_PAIR_R("2", "3", R, "d1")                  \
  DV_NORM2_PAIR_R("4", "5", R, "d2") DV_NORM2_PAIR_R("6", "7", R, "d3") DV_NORM2_PAIR_R("8", "9", R, "d4")          \
  DV_NORM2_PAIR_R("10", "11", R, "d5") DV_NORM2_PAIR_R("12", "13", R, "d6") DV_NORM2_PAIR_R("14", "15", R, "d7") "}"
#define DV_TREE16R(OP2, SLOT, R)                                                                                   \
  "{\n\t.reg .b32 r<8>;\n\t.reg .pred p;\n\t"                                                                      \
  OP2("r0", R "0", R "1") OP2("r1", R "2", R "3") OP2("r2", R "4", R "5") OP2("r3", R "6", R "7")                  \
  OP2("r4", R "8", R "9") OP2("r5", R "10", R "11") OP2("r6", R "12", R "13") OP2("r7", R "14", R "15")            \
  OP2("r0", "r0", "r1") OP2("r2", "r2", "r3") OP2("r4", "r4", "r5") OP2("r6", "r6", "r7")                          \
  OP2("r0", "r0", "r2") OP2("r4", "r4", "r6") OP2("r0", "r0", "r4") OP2("vp" SLOT, "vp" SLOT, "r0") "}"

// ---- lane templates ----------------------------------------------------------------------------------
#define DV_BINV_LANE(i, OP) OP " va" #i ", va" #i ", vb" #i ";\n\t"
#define DV_RBINV_LANE(i, OP) OP " va" #i ", vb" #i ", va" #i ";\n\t"
#define DV_BINS_LANE(i, OP) OP " va" #i ", va" #i ", %0;\n\t"
#define DV_RBINS_LANE(i, OP) OP " va" #i ", %0, va" #i ";\n\t"
#define DV_PICKV_LANE(i, SETP) SETP " p, va" #i ", vb" #i ";\n\tselp.b32 va" #i ", va" #i ", vb" #i ", p;\n\t"
#define DV_PICKS_LANE(i, SETP) SETP " p, va" #i ", %0;\n\tselp.b32 va" #i ", va" #i ", %0, p;\n\t"
#define DV_SQR_LANE(i, X) "mul.f32 va" #i ", va" #i ", va" #i ";\n\t"
#define DV_UN_LANE(i, OP) OP " va" #i ", va" #i ";\n\t"
#define DV_EXPF_LANE(i, X) "mul.f32 va" #i ", va" #i ", 0f3FB8AA3B;\n\tex2.approx.ftz.f32 va" #i ", va" #i ";\n\t"
#define DV_ISFIN_LANE(i, X) "testp.finite.f32 p, va" #i ";\n\tselp.b32 va" #i ", 0x3f800000, 0, p;\n\t"
#define DV_RNDH_LANE(i, X) "cvt.rn.f16.f32 h, va" #i ";\n\tcvt.f32.f16 va" #i ", h;\n\t"
#define DV_RNDB_PAIR(a, b, X) "cvt.rn.bf16x2.f32 t, va" b ", va" a ";\n\tshl.b32 va" a ", t, 16;\n\tand.b32 va" b ", t, 0xffff0000;\n\t"
#define DV_CMPF_LANE(i, SETP) SETP " p, va" #i ", vb" #i ";\n\tselp.b32 va" #i ", 0x3f800000, 0, p;\n\t"
#define DV_CMPI_LANE(i, SETP) SETP " p, va" #i ", vb" #i ";\n\tselp.b32 va" #i ", 1, 0, p;\n\t"
#define DV_PRED_LANE(i, TEST, ZERO) TEST #i ZERO ";\n\tselp.u32 t, 1, 0, p;\n\tbfi.b32 %0, t, %0, " #i ", 1;\n\t"
#define DV_SELM_LANE(i, X) "bfe.u32 t, %0, " #i ", 1;\n\tsetp.ne.u32 p, t, 0;\n\tselp.b32 va" #i ", va" #i ", vb" #i ", p;\n\t"
#define DV_NEZ_LANE(i, TEST, ZERO) TEST #i ZERO ";\n\tselp.b32 va" #i ", 1, 0, p;\n\t"
#define DV_MOV_LANE(i, D, S_) "mov.b32 " D #i ", " S_ #i ";\n\t"
#define DV_GETLANE(i, R) "mov.b32 %" #i ", " R #i ";\n\t"
#define DV_SETLANE(i, R) "mov.b32 " R #i ", %" #i ";\n\t"
#define DV_SPLATLANE(i, R) "mov.b32 " R #i ", %0;\n\t"
// fused handlers: two operations on a lane, each rounded on its own (.rn keeps ptxas from contracting them into an fma)
#define DV_BINS2_LANE(i, OP1, OP2) OP1 " va" #i ", va" #i ", %0;\n\t" OP2 " va" #i ", va" #i ", %1;\n\t"
#define DV_BINS3_LANE(i, OP1, OP2, OP3) \
  OP1 " va" #i ", va" #i ", %0;\n\t" OP2 " va" #i ", va" #i ", %1;\n\t" OP3 " va" #i ", va" #i ", %2;\n\t"
#define DV_NORM_LANE(i, X)                                                                                  \
  "sub.rn.f32 va" #i ", va" #i ", %0;\n\tmul.rn.f32 va" #i ", va" #i ", %1;\n\tmul.rn.f32 va" #i ", va" #i ", %2;\n\t" \
  "add.rn.f32 va" #i ", va" #i ", %3;\n\t"
#define DV_CSQR_LANE(i, X) "sub.rn.f32 va" #i ", va" #i ", %0;\n\tmul.rn.f32 va" #i ", va" #i ", va" #i ";\n\t"
#define DV_BINVRN_LANE(i, OP) OP " va" #i ", va" #i ", vb" #i ";\n\t"
#define DV_SQRRN_LANE(i, X) "mul.rn.f32 va" #i ", va" #i ", va" #i ";\n\t"
#define DV_SIGM_LANE(i, X)                                                                                  \
  "mul.rn.f32 va" #i ", va" #i ", 0fBF800000;\n\tmul.rn.f32 va" #i ", va" #i ", 0f3FB8AA3B;\n\t"            \
  "ex2.approx.ftz.f32 va" #i ", va" #i ";\n\tadd.rn.f32 va" #i ", va" #i ", 0f3F800000;\n\trcp.approx.ftz.f32 va" #i ", va" #i ";\n\t"
// packed f32x2 forms of the fused handlers' arithmetic: two neighbouring lanes of va (and of vb) travel as one 64-bit
// pair, one instruction works on both.  Only where no addition follows a multiplication directly in packed form (the
// assembler contracts that pair into a fused multiply-add, which rounds once instead of twice).
#define DV_PAIRS8V(M, X)                                                                                          \
  "{\n\t.reg .b64 d<8>, e<8>;\n\t" M("0", "1", "d0", "e0", X) M("2", "3", "d1", "e1", X) M("4", "5", "d2", "e2", X)   \
  M("6", "7", "d3", "e3", X) M("8", "9", "d4", "e4", X) M("10", "11", "d5", "e5", X) M("12", "13", "d6", "e6", X)    \
  M("14", "15", "d7", "e7", X) "}"
#define DV_P2_PACKAB(a, b, D, E) "mov.b64 " D ", {va" a ", va" b "};\n\tmov.b64 " E ", {vb" a ", vb" b "};\n\t"
#define DV_P2_UNPACK(a, b, D) "mov.b64 {va" a ", va" b "}, " D ";\n\t"
// va <- (va + vb)^2
#define DV_P2_ADDSQR(a, b, D, E, X)                                                                               \
  DV_P2_PACKAB(a, b, D, E) "add.rn.f32x2 " D ", " D ", " E ";\n\tmul.rn.f32x2 " D ", " D ", " D ";\n\t" DV_P2_UNPACK(a, b, D)
// va <- (va + vb) * scalar pair %0
#define DV_P2_ADDMULS(a, b, D, E, X)                                                                              \
  DV_P2_PACKAB(a, b, D, E) "add.rn.f32x2 " D ", " D ", " E ";\n\tmul.rn.f32x2 " D ", " D ", %0;\n\t" DV_P2_UNPACK(a, b, D)
// va <- va OP vb
#define DV_P2_BINV(a, b, D, E, OP) DV_P2_PACKAB(a, b, D, E) OP " " D ", " D ", " E ";\n\t" DV_P2_UNPACK(a, b, D)
// va <- 1 / (1 + 2^(va * -log2(e)))   (%0 = the pair of -log2(e), %1 = the pair of 1.0; x * -1 is exact, so one
// multiplication by -log2(e) gives the bits of (x * -1) * log2(e))
#define DV_P2_SIGM(a, b, D, E, X)                                                                                 \
  "mov.b64 " D ", {va" a ", va" b "};\n\tmul.rn.f32x2 " D ", " D ", %0;\n\t" DV_P2_UNPACK(a, b, D)                     \
  "ex2.approx.ftz.f32 va" a ", va" a ";\n\tex2.approx.ftz.f32 va" b ", va" b ";\n\t"                                 \
  "mov.b64 " D ", {va" a ", va" b "};\n\tadd.rn.f32x2 " D ", " D ", %1;\n\t" DV_P2_UNPACK(a, b, D)                     \
  "rcp.approx.ftz.f32 va" a ", va" a ";\n\trcp.approx.ftz.f32 va" b ", va" b ";\n\t"
// tree reductions of the 16 accumulator lanes into partial register vp<SLOT>
#define DV_TREE16(OP2, SLOT)                                                                                       \
  "{\n\t.reg .b32 r<8>;\n\t.reg .pred p;\n\t"                                                                      \
  OP2("r0", "va0", "va1") OP2("r1", "va2", "va3") OP2("r2", "va4", "va5") OP2("r3", "va6", "va7")                  \
  OP2("r4", "va8", "va9") OP2("r5", "va10", "va11") OP2("r6", "va12", "va13") OP2("r7", "va14", "va15")            \
  OP2("r0", "r0", "r1") OP2("r2", "r2", "r3") OP2("r4", "r4", "r5") OP2("r6", "r6", "r7")                          \
  OP2("r0", "r0", "r2") OP2("r4", "r4", "r6") OP2("r0", "r0", "r4") OP2("vp" SLOT, "vp" SLOT, "r0") "}"
#define DV_ADD2(D, A, B) "add.f32 " D ", " A ", " B ";\n\t"
#define DV_MAX2(D, A, B) "setp.gt.f32 p, " A ", " B ";\n\tselp.b32 " D ", " A ", " B ", p;\n\t"
#define DV_MIN2(D, A, B) "setp.lt.f32 p, " A ", " B ";\n\tselp.b32 " D ", " A ", " B ", p;\n\t"
#define DV_ADDRN2(D, A, B) "add.rn.f32 " D ", " A ", " B ";\n\t"
#define DV_SUM_TREE(SLOT) DV_TREE16(DV_ADD2, SLOT)
#define DV_SUMRN_TREE(SLOT) DV_TREE16(DV_ADDRN2, SLOT)
#define DV_MAX_TREE(SLOT) DV_TREE16(DV_MAX2, SLOT)
#define DV_MIN_TREE(SLOT) DV_TREE16(DV_MIN2, SLOT)

// ---- whole-register operations ---------------------------------------------------------------------------
#define DV_OUT16(X)                                                                                                   \
  "=r"(X[0]), "=r"(X[1]), "=r"(X[2]), "=r"(X[3]), "=r"(X[4]), "=r"(X[5]), "=r"(X[6]), "=r"(X[7]), "=r"(X[8]),         \
    "=r"(X[9]), "=r"(X[10]), "=r"(X[11]), "=r"(X[12]), "=r"(X[13]), "=r"(X[14]), "=r"(X[15])
#define DV_IN16(X)                                                                                                    \
  "r"(X[0]), "r"(X[1]), "r"(X[2]), "r"(X[3]), "r"(X[4]), "r"(X[5]), "r"(X[6]), "r"(X[7]), "r"(X[8]), "r"(X[9]),       \
    "r"(X[10]), "r"(X[11]), "r"(X[12]), "r"(X[13]), "r"(X[14]), "r"(X[15])
#define DV_GET(R, X) asm volatile(DV_LN(DV_GETLANE, R) : DV_OUT16(X));
#define DV_SET(R, X) asm volatile(DV_LN(DV_SETLANE, R)::DV_IN16(X));
#define DV_SPLAT(R, V) asm volatile(DV_LN(DV_SPLATLANE, R)::"r"(V));

// four 16-byte granules from shared memory (fp32 / int32 tensors, temporaries)
#define DV_LDR32(R, A0, A1, A2, A3)                                                \
  asm volatile("ld.shared.v4.b32 {" R "0," R "1," R "2," R "3}, [%0];\n\t"         \
               "ld.shared.v4.b32 {" R "4," R "5," R "6," R "7}, [%1];\n\t"         \
               "ld.shared.v4.b32 {" R "8," R "9," R "10," R "11}, [%2];\n\t"       \
               "ld.shared.v4.b32 {" R "12," R "13," R "14," R "15}, [%3];" ::"r"(A0), \
               "r"(A1), "r"(A2), "r"(A3)                                           \
               : "memory");
#define DV_LD16_RAW                                                                                       \
  "ld.shared.v2.b32 {t0,t1}, [%0];\n\tld.shared.v2.b32 {t2,t3}, [%1];\n\tld.shared.v2.b32 {t4,t5}, [%2];\n\t" \
  "ld.shared.v2.b32 {t6,t7}, [%3];\n\t"
#define DV_BF16_PAIR(R, a, b, T) "shl.b32 " R a ", " T ", 16;\n\tand.b32 " R b ", " T ", 0xffff0000;\n\t"
#define DV_LDR_BF16(R, A0, A1, A2, A3)                                                                          \
  asm volatile("{\n\t.reg .b32 t0, t1, t2, t3, t4, t5, t6, t7;\n\t" DV_LD16_RAW                                 \
               DV_BF16_PAIR(R, "0", "1", "t0") DV_BF16_PAIR(R, "2", "3", "t1") DV_BF16_PAIR(R, "4", "5", "t2")   \
               DV_BF16_PAIR(R, "6", "7", "t3") DV_BF16_PAIR(R, "8", "9", "t4") DV_BF16_PAIR(R, "10", "11", "t5") \
               DV_BF16_PAIR(R, "12", "13", "t6") DV_BF16_PAIR(R, "14", "15", "t7") "}" ::"r"(A0),                \
               "r"(A1), "r"(A2), "r"(A3)                                                                        \
               : "memory");
#define DV_F16_PAIR(R, a, b, T) "mov.b32 {h0,h1}, " T ";\n\tcvt.f32.f16 " R a ", h0;\n\tcvt.f32.f16 " R b ", h1;\n\t"
#define DV_LDR_F16(R, A0, A1, A2, A3)                                                                          \
  asm volatile("{\n\t.reg .b32 t0, t1, t2, t3, t4, t5, t6, t7;\n\t.reg .b16 h0, h1;\n\t" DV_LD16_RAW            \
               DV_F16_PAIR(R, "0", "1", "t0") DV_F16_PAIR(R, "2", "3", "t1") DV_F16_PAIR(R, "4", "5", "t2")     \
               DV_F16_PAIR(R, "6", "7", "t3") DV_F16_PAIR(R, "8", "9", "t4") DV_F16_PAIR(R, "10", "11", "t5")   \
               DV_F16_PAIR(R, "12", "13", "t6") DV_F16_PAIR(R, "14", "15", "t7") "}" ::"r"(A0),                 \
               "r"(A1), "r"(A2), "r"(A3)                                                                       \
               : "memory");
#define DV_U8_QUAD(R, a, b, c, d, T) \
  "and.b32 " R a ", " T ", 255;\n\tbfe.u32 " R b ", " T ", 8, 8;\n\tbfe.u32 " R c ", " T ", 16, 8;\n\tshr.u32 " R d ", " T ", 24;\n\t"
#define DV_LDR_U8(R, A0, A1, A2, A3)                                                                             \
  asm volatile("{\n\t.reg .b32 t0, t1, t2, t3;\n\tld.shared.b32 t0, [%0];\n\tld.shared.b32 t1, [%1];\n\t"         \
               "ld.shared.b32 t2, [%2];\n\tld.shared.b32 t3, [%3];\n\t"                                          \
               DV_U8_QUAD(R, "0", "1", "2", "3", "t0") DV_U8_QUAD(R, "4", "5", "6", "7", "t1")                   \
               DV_U8_QUAD(R, "8", "9", "10", "11", "t2") DV_U8_QUAD(R, "12", "13", "14", "15", "t3") "}" ::"r"(A0), \
               "r"(A1), "r"(A2), "r"(A3)                                                                         \
               : "memory");

// run FN("va" | "vb", args...) for destination code D
#define DV_BY_DEST(D, FN, ...)                \
  {                                           \
    const uint32_t d_ = (D);                  \
    if (d_ == UD_ACC) { FN("va", __VA_ARGS__) } else { FN("vb", __VA_ARGS__) } \
  }
#define DV_BIN_CASES(K, VLANE, SLANE, OP)                                      \
  case UH_BINV_FIRST + K: asm volatile(DV_LN(VLANE, OP)); break;               \
  case UH_BINS_FIRST + K: asm volatile(DV_LN(SLANE, OP)::"r"(uhi)); break;     \
  case UH_BINR_FIRST + K: {                                                    \
    const uint32_t sv_ = lds32(sreg_addr(arg));                                \
    asm volatile(DV_LN(SLANE, OP)::"r"(sv_));                                  \
    break;                                                                     \
  }
#define DV_CMP_ASM(LANE, SETP) asm volatile("{\n\t.reg .pred p;\n\t" DV_LN(LANE, SETP) "}")

#endif  // DVM_B200_VM_VECTOR_REGS_H_
