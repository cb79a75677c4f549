// The one-launch quantised transformer-encoder evaluator for sm_100a, and its C ABI.
//
// What one launch computes (per position): embedding of 32 piece words, 8 pre-norm
// encoder layers of width 256 (8 heads of 32, FFN 1024) with every weight GEMM in
// s8/u8 x s8 -> s32 on the tcgen05 tensor cores, a final LayerNorm, and the fp16 head
// product giving 32x64 policy logits, 32x4 promotion logits and the value; optionally the
// search node's edges and priors straight from the epilogue.  The int8 arithmetic follows
// the reference kernel (csrc/encoder.cu:1225-1599 with int8_gemm.cuh) at every rounding
// point, the hardware-approximate ones included (summation order and 1/sqrt of the norms,
// fp16 accumulation in the attention and head products, __expf), so that its outputs equal
// that kernel's bit for bit.  The weight GEMMs and the head product run on tcgen05 (exact
// integers; fp16 x fp16 with fp16 accumulators, which carries the bits of the reference's
// fp16-accumulate mma.sync); the 32 x 32 attention products run as mma.sync on the row warps.
//
// Shape of the kernel
//   * persistent grid, one CTA per SM, each CTA loops over tiles of 128 token rows
//     (4 boards);
//   * 19 warps: 16 "row" warps, one weight-stream producer, two MMA issuers;
//   * row warps: thread = (row, quarter).  Warp w works on TMEM lanes 32*(w%4)..+31, i.e.
//     on board w%4 of the tile, and on quarter w/4 of each row's columns.  All LayerNorm /
//     quantise / descale work is thread-local plus one exchange among the four quarters;
//     the four warps of a board synchronise with a 128-thread named barrier, and the four
//     boards of a tile never wait for one another except through the shared MMA;
//   * weights never sit in shared memory for longer than one use: the host packs them
//     as ready-made 128-byte-swizzled K-major stage images and the producer streams
//     them through a ring with cp.async.bulk + mbarrier;
//   * accumulators live in tensor memory: columns [0,128) hold the fp16 residual
//     stream x (two halves per column), [128,256) the attention output / the FFN's fp16
//     running total, [256,512) the GEMM accumulators.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>
#include <new>
#include <string>

#include "../../include/brokefish_b200.h"
#include "bf_movegen.cuh"
#include "bf_ptx.cuh"

namespace bf {
using namespace bfptx;

constexpr int kD = 256, kDFF = 1024, kT = 32, kRows = 128;
constexpr int kRowWarps = 16, kProducerWarp = 16, kMmaWarp = 17, kMmaWarp2 = 18, kThreads = 608;
constexpr int kLparamStride = 4736;
constexpr int LP_SW_QKV = 0, LP_SW_O = 24, LP_SW_FF1 = 32, LP_SW_FF2 = 64;
constexpr int LP_B_QKV = 128, LP_B_O = 1664, LP_B_FF1 = 2176, LP_B_FF2 = 4224;
constexpr int EMB_SQUARE = 0, EMB_TS = 64, EMB_CT = 76, EMB_CLOCK = 80, EMB_REP = 181;
constexpr int kNClock = 101, kNRep = 3, kNTypeSpecial = 12;

// ---- shared memory map (offsets from a 1024-byte aligned base) ----------------------
// Arithmetic of a kernel arm: which formats the weight GEMMs run in.
//   kArInt8  every weight GEMM s8/u8 x s8 -> s32 (the reference's int8 "all" scheme)
//   kArE4M3  FFN e4m3 x e4m3, QKV and out-projection fp16 x fp16 (the reference's fp8 path)
//   kArF16   every weight GEMM fp16 x fp16 with fp16 accumulators (the reference's default path)
//   kArI8Ffn FFN s8/u8 x s8 as in kArInt8, QKV and out-projection fp16 x fp16 as in kArF16 (the
//            reference's "ffn" int8 scheme, quant 2)
//   kArI8Qkv FFN and QKV s8 x s8, out-projection fp16 x fp16 (the reference's "ffn+qkv" int8
//            scheme, quant 4)
enum { kArInt8 = 0, kArE4M3 = 1, kArF16 = 2, kArI8Ffn = 3, kArI8Qkv = 4 };
// The front of the map depends on the arithmetic.  int8: the A operand is 32 KB of bytes and
// the weight ring has 112 KB.  With fp16 attention GEMMs (e4m3, fp16 arms) the A operand is 64 KB
// (4 K-slabs of 64 halves) and the ring gives up two slots.
template <int kAr>
struct Cfg {
    static constexpr bool kHalfA = kAr != kArInt8;           // the A operand region holds fp16 K-slabs
    static constexpr bool kQkvF16 = kAr == kArE4M3 || kAr == kArF16 || kAr == kArI8Ffn;   // fp16 QKV GEMM
    static constexpr bool kOutF16 = kHalfA;                  // fp16 out-projection GEMM
    static constexpr uint32_t SM_A = 0;     // A operand: K-slabs of [128 rows][128 B]
    static constexpr uint32_t SM_R = kHalfA ? 65536 : 32768; // 64 KB: Q/K/V staging (3 x 16 KB) |
                                            // hidden operand(s) | fp16 head A (4 x 16 KB)
    static constexpr uint32_t SM_RING = SM_R + 65536;        // weight ring up to SM_XCH
    static constexpr int kQSlots = kHalfA ? 3 : 4;           // 24 KB QKV stages
    static constexpr int kRSlots = kHalfA ? 5 : 7;           // 16 KB stages
    static constexpr int kQkvSlabs = kQkvF16 ? 4 : 2;        // K-slabs of a QKV unit
    static constexpr int kOutSlabs = kOutF16 ? 4 : 2;        // K-slabs of an out-projection unit
    static constexpr int kFfnSlabs = kAr == kArF16 ? 4 : 2;  // K-slabs of an FFN unit
    static constexpr int kLayerStream = kAr == kArF16 ? 1572864
                                      : (kAr == kArE4M3 || kAr == kArI8Ffn) ? 1048576
                                      : kAr == kArI8Qkv ? 851968 : 786432;
};
constexpr uint32_t SM_XCH = 212992;     // 16 KB: float4 [2 parity][4 quarter][128 rows]
constexpr uint32_t SM_BAR = 229376;     // mbarriers
constexpr uint32_t SM_MISC = SM_BAR + 256;
constexpr uint32_t SM_PROF = SM_MISC + 64;     // 16 x int64 phase cycle counters
constexpr uint32_t SM_BYTES = SM_PROF + 128;
constexpr uint32_t kSmemRequest = SM_BYTES + 1024;
constexpr uint32_t kQStage = 24576, kRStage = 16384;
// the weight stream ends with the [96 x 256] fp16 head matrix as 4 K-slabs of [96 rows][128 B]
constexpr uint32_t kHeadStage = 12288, kHeadStages = 4;
// tail section: gamma, beta and three value rows of the final norm / value head (1280 halves)
constexpr uint32_t kTailBytes = 2560u;
// barrier indices
constexpr int B_WQ_FULL = 0, B_WQ_EMPTY = 4, B_WR_FULL = 8, B_WR_EMPTY = 15, B_ACC_FULL = 22,
              B_ACC_EMPTY = 24, B_A_READY = 26, B_A2_READY = 27, B_COUNT = 29;
// ---- tensor memory map (columns) ---------------------------------------------------------
constexpr uint32_t TM_X = 0, TM_OY = 128, TM_ACC = 256, TM_COLS = 512;

// time-out codes written to the status word (which wait gave up)
enum { kErrProducer = 1, kErrMmaOperand = 2, kErrMmaWeights = 3, kErrMmaAcc = 4, kErrRowAcc = 5 };

// Ranges of the quantised operands: a row's (or a 128-output weight block's) scale is its
// largest magnitude over these (int8_gemm.cuh:26-30, 98, 166: signed 127, unsigned 255;
// fp8_gemm.cuh: the e4m3 operands are scaled into +-8).
constexpr float kQMaxS8 = 127.0f, kQMaxU8 = 255.0f, kQMaxE4M3 = 8.0f;

struct Params {
    const uint16_t* boards;
    const int16_t* control;
    const uint8_t* rep;
    const uint64_t* legal;
    int n, n_layers, n_value, vmode;
    int quant;                  // 3 = int8 on all four matmuls, 2 = int8 FFN only, 4 = int8 FFN and QKV,
                                // 1 = e4m3 FFN, 0 = fp16 (the reference's numbering)
    int rsqrt_rn;               // 1: correctly rounded 1/sqrt in the norms (what a CPU can reproduce);
                                // 0: the hardware approximation, as the reference's rsqrtf (encoder.cu:597)
    float eps;
    float one;                  // 1.0f (see quant16)
    const uint8_t* wstream;
    const uint8_t* lparams;
    const __half* emb;
    const __half* tail;
    const __half* rj;           // re-injection coefficients [sites][8] or null
    int rj_mode;                // 0 none, 1 attention norms, 2 both norms
    __half* policy;
    __half* promo;
    float* value;
    __half* y;
    // fused expansion (optional): per position up to `e_cap` edges in canonical order
    __half* prior;              // [n, e_cap] fp16 priors, zero beyond the edge count
    int16_t* move;              // [n, e_cap] labels: slot * 64 + square | promotion type << 11
    int* nedges;                // [n] edges written
    int e_cap;
    int debug_stage, debug_layer;
    int cap_layer, cap_op;
    uint8_t* cap_a;
    int32_t* cap_acc;
    // backbone-only entry (instrumented arm): activations in instead of the embedding, optional
    // per-token alive flags instead of the piece words' captured bit
    const __half* x_in;
    const int8_t* alive_in;
    // compacted leaf list (optional): evaluate positions leaf_index[0 .. *leaf_count) of the
    // staged arrays; `n` is then the capacity (the most the list can hold) the grid was sized for
    const int* leaf_index;
    const int* leaf_count;
    int* status;
    unsigned long long* prof;   // 16 phase counters (cycles of warp 0, lane 0 of every CTA) or null
};

// Per-thread context of a row warp.  Sixteen row warps: warp w works on TMEM lanes
// 32*(w%4)..+31 (board w%4 of the tile) and on quarter w/4 of each row's columns.
struct RowCtx {
    int lane, q, qt, row;       // q: board within the tile, qt: which quarter of the columns
    uint32_t smem;              // shared base (shared-space address)
    uint32_t sm_a, sm_r;        // A operand and the 64 KB staging / hidden / head-operand region
    uint8_t* smem_gen;          // shared base (generic pointer)
    uint32_t tm;                // TMEM base address with this warp's lane offset
    volatile int* abort_flag;
    int xpar;                   // exchange buffer parity
    uint64_t one2;              // (1.0f, 1.0f) from the launch parameters, opaque to the compiler
    uint32_t full0, full1;      // accumulator slots consumed so far
    long grow;                  // global token row = board * 32 + token
    int n;                      // positions this launch evaluates (the leaf count when a list is given)
    bool valid;                 // this warp's board exists
    uint32_t word;              // this token's piece word
    int stm, clk, rp;           // board-level embedding indices (side to move, clock, repetition)
    bool prof_on;               // this thread keeps the CTA's phase clock
    long long t_last;
};

// In-kernel phase accounting (the counterpart of the reference's prof::Timer,
// csrc/encoder.cu:1110-1177): one thread per CTA charges the cycles since its previous mark to
// a phase.  Off (one predictable branch per mark) unless the launch carries a counter buffer.
enum { PH_EMBED = 0, PH_LN, PH_WAIT_MMA, PH_QKV_EPI, PH_PAIR_BAR, PH_ATTENTION, PH_O_READBACK, PH_O_QUANT,
       PH_OUT_EPI, PH_FF1_EPI, PH_FF2_EPI, PH_HEAD, PH_WAIT_OUT, PH_WAIT_FF1, PH_WAIT_FF2, PH_WAIT_FF1_FIRST,
       PH_COUNT };
template <bool kDbg>
__device__ __forceinline__ void prof_mark(RowCtx& c, int phase) {
    if (kDbg && c.prof_on) {
        const long long t = clock64();
        long long* a = reinterpret_cast<long long*>(c.smem_gen + SM_PROF);
        a[phase] += t - c.t_last;
        c.t_last = t;
    }
}

__device__ __forceinline__ uint32_t bar_addr(uint32_t smem, int idx) {
    return smem + SM_BAR + 8u * idx;
}

// The four warps of a board meet here (named barrier 1 + board, 128 threads).
__device__ __forceinline__ void board_sync(const RowCtx& c) { named_bar_sync(1 + c.q, 128); }

// Exchange one float4 among the four threads that share a row; `all[k]` is quarter k's.
__device__ __forceinline__ void exchange4(RowCtx& c, float4 mine, float4 (&all)[4]) {
    const uint32_t xch = c.smem + SM_XCH + 16u * (c.xpar * 4 * kRows + c.row);
    sts_f4(xch + 16u * kRows * c.qt, mine);
    board_sync(c);
#pragma unroll
    for (int k = 0; k < 4; ++k) all[k] = lds_f4(xch + 16u * kRows * k);
    c.xpar ^= 1;
}
__device__ __forceinline__ float exchange_max(RowCtx& c, float mine) {
    float4 all[4];
    exchange4(c, make_float4(mine, 0.f, 0.f, 0.f), all);
    return fmaxf(fmaxf(all[0].x, all[1].x), fmaxf(all[2].x, all[3].x));
}

template <bool kDbg>
__device__ __forceinline__ void row_wait_acc(RowCtx& c, int slot, int phase_before, int phase_wait = PH_WAIT_MMA) {
    prof_mark<kDbg>(c, phase_before);
    const uint32_t n = slot ? c.full1 : c.full0;
    mbar_wait(bar_addr(c.smem, B_ACC_FULL + slot), n & 1, c.abort_flag, kErrRowAcc);
    if (slot) c.full1 = n + 1; else c.full0 = n + 1;
    tc_fence_after();
    prof_mark<kDbg>(c, phase_wait);
}
// All of this warp's TMEM loads of the slot are done: hand it back to the MMA issuer.
__device__ __forceinline__ void row_release_acc(RowCtx& c, int slot) {
    tmem_wait_ld();
    tc_fence_before();
    __syncwarp();
    if (c.lane == 0) mbar_arrive(bar_addr(c.smem, B_ACC_EMPTY + slot));
}
// This warp's generic-proxy writes of an MMA operand are done: publish to the issuer.
__device__ __forceinline__ void row_publish(RowCtx& c, int bar_idx) {
    fence_proxy_async_smem();
    __syncwarp();
    if (c.lane == 0) mbar_arrive(bar_addr(c.smem, bar_idx));
}

// Round-half-even float -> 8-bit integer in the low byte (two's complement for
// negatives): adding 1.5 * 2^23 leaves the integer in the low mantissa bits.  Same
// result as `cvt.rni.sat` for |v| <= 255 (int8_gemm.cuh:190-199 guarantees the range).
__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// 8 packed fp16 pairs (16 values) -> 16 quantised bytes: fp32 multiply by 1/scale, then the
// rounding add, two lanes at a time.
// `one2` is 1.0 in both lanes, read from the launch parameters so that the compiler cannot see
// its value: the rounding add is written as fma(x, 1, magic), and with a literal 1 the product
// `x = h * inv` was fused into it, skipping the rounding of the product the scheme specifies.
__device__ __forceinline__ uint4 quant16(const uint32_t* h, float inv, uint64_t one2) {
    const uint64_t inv2 = pk2(inv, inv), magic2 = pk2(12582912.0f, 12582912.0f);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float a0, a1, b0, b1;
        upk2(fma2(mul2(h2_to_f2(h[2 * k]), inv2), one2, magic2), a0, a1);
        upk2(fma2(mul2(h2_to_f2(h[2 * k + 1]), inv2), one2, magic2), b0, b1);
        o[k] = pack4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(b0), __float_as_uint(b1));
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// The e4m3 twin: the scaled value is rounded to fp16 first, then to e4m3, as the reference's
// quantiser does (csrc/fp8_gemm.cuh:186-199); low half to the low byte.
__device__ __forceinline__ uint4 quant16_e4m3(const uint32_t* h, float inv) {
    const uint64_t inv2 = pk2(inv, inv);
    uint32_t o[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = e4m3x2_from_h2(f2_to_h2(mul2(h2_to_f2(h[2 * k]), inv2)));
        const uint32_t hi = e4m3x2_from_h2(f2_to_h2(mul2(h2_to_f2(h[2 * k + 1]), inv2)));
        o[k] = lo | (hi << 16);
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
template <bool kFP8>
__device__ __forceinline__ uint4 quant16_any(const uint32_t* h, float inv, uint64_t one2) {
    if (kFP8) return quant16_e4m3(h, inv);
    return quant16(h, inv, one2);
}
// Address of 16-byte group `chunk` of row `row` in a [rows][128 B] swizzled tile.
__device__ __forceinline__ uint32_t sw_off(int row, int chunk) {
    return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

// `(float(acc) * sa) * sw` -> fp16, + fp16 bias, optional ReLU; kN columns -> kN/2 pairs
// (int8_gemm.cuh:276-297, encoder.cu:631-644, 1482-1489).
// kAcc says what the accumulator holds: kAccInt = s32 with the two scales, kAccFloat = fp32
// with the two scales (e4m3 GEMMs; csrc/fp8_gemm.cuh:288-310), kAccPlain = the fp16 accumulator
// of an fp16 GEMM, one value in the low half of each word, no scales (the reference's
// un-quantised QKV / out-projection, whose mma.sync accumulates in fp16; tcgen05 kind::f16 with
// fp16 accumulators gives the same bits).
enum { kAccInt = 0, kAccFloat = 1, kAccPlain = 2 };
template <int kN, bool kRelu, int kAcc = kAccInt>
__device__ __forceinline__ void descale(const uint32_t* acc, float sa, float sw, const __half* bias,
                                        uint32_t* out) {
    const uint4* b4 = reinterpret_cast<const uint4*>(bias);
    const uint64_t sa2 = pk2(sa, sa), sw2 = pk2(sw, sw);
#pragma unroll
    for (int v = 0; v < kN / 8; ++v) {
        const uint4 bv = __ldg(b4 + v);
        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int i = 4 * v + k;
            // exact s32 -> f32 on the conversion unit (otherwise idle here; the integer-add
            // form measured 6 % slower because it loads the FMA pipe, which is the busy one),
            // then the two fp32 multiplies
            if (kAcc == kAccPlain) {
                const uint32_t h = __byte_perm(acc[2 * i], acc[2 * i + 1], 0x5410);
                out[i] = kRelu ? hfma2_relu(h, 0x3C003C00u, bw[k]) : as_u32(__hadd2(as_h2(h), as_h2(bw[k])));
                continue;
            }
            // the row-scale multiply as two scalar multiplies (they spread over both halves of
            // the fp32 pipe; measured 0.5 % faster than the packed form), the weight-scale one packed
            uint64_t f;
            if (kAcc == kAccInt)
                f = pk2(__fmul_rn(static_cast<float>(static_cast<int>(acc[2 * i])), sa),
                        __fmul_rn(static_cast<float>(static_cast<int>(acc[2 * i + 1])), sa));
            else
                f = mul2(pk2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1])), sa2);
            f = mul2(f, sw2);
            if (kRelu) {
                // relu(x + b) in one instruction: x * 1 is exact, so the sum is rounded once
                // exactly as the fp16 add is, and the clamp is part of the same operation
                out[i] = hfma2_relu(f2_to_h2(f), 0x3C003C00u, bw[k]);
            } else {
                out[i] = as_u32(__hadd2(as_h2(f2_to_h2(f)), as_h2(bw[k])));
            }
        }
    }
}

template <int kN>
__device__ __forceinline__ float amax_h2(const uint32_t* h, bool take_abs) {
    __half2 m = __float2half2_rn(0.0f);
#pragma unroll
    for (int i = 0; i < kN; ++i) {
        const __half2 v = as_h2(h[i]);
        m = __hmax2(m, take_abs ? __habs2(v) : v);
    }
    return fmaxf(__low2float(m), __high2float(m));
}

template <int kN>
__device__ __forceinline__ void store_words(void* dst, const uint32_t* w) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int k = 0; k < kN / 4; ++k) d4[k] = make_uint4(w[4 * k], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
}

// One LayerNorm of the residual stream (TMEM) for this thread's quarter row (columns
// 32*qt + [0,32) and 128 + 32*qt + [0,32)), in two passes, followed either by the s8
// quantisation into the A operand (returns the row scale) or, for the final norm, by the
// affine and the fp16 store into the head product's A operand.
//
// Statistics: fp32, one pass, variance clamped at zero, in the reference's own summation
// order (encoder.cu:566-598; the CPU oracle mirrors it): eight contiguous columns summed one
// after the other, then the 32 partial sums combined by the butterfly 16, 8, 4, 2, 1.  1/sqrt
// is the hardware approximation the reference uses, or correctly rounded when the launch asks
// for it (`rsqrt_rn`, the only form a CPU can reproduce).  x_hat = fp16((x - mean) * rstd).
//
// Quantisation (int8_gemm.cuh:159-199): scale = amax(x_hat)/127, all-zero row -> 1.  The map
// x -> x_hat is monotone (every rounding in it is), so amax(x_hat) is reached at the row's
// largest or smallest x and needs no second pass: the row minimum and maximum travel in the
// same exchange as the sums.
// Per-layer input re-injection (csrc/encoder.cu:384-416, 439-583): what the LayerNorm is given
// is `x + sum_k c[site][k] * E_k` with the five embedding rows of this token, in the
// reference's fp16 order: pb = fma(c_clk, clock, c_rep * rep); cs = fma(c_ct, color_turn by
// *slot* colour, pb); then fma(c_ts, type_special, fma(c_sq, square, x)) + cs.  The residual
// stream itself is not touched.  32 columns starting at `col`.
__device__ __forceinline__ void reinject32(const RowCtx& c, const Params& p, int site, int col,
                                           uint32_t (&x)[16]) {
    const uint4 cf = __ldg(reinterpret_cast<const uint4*>(p.rj + site * 8));
    const __half2 c_sq = __half2half2(__low2half(as_h2(cf.x))), c_ts = __half2half2(__high2half(as_h2(cf.x)));
    const __half2 c_ct = __half2half2(__low2half(as_h2(cf.y))), c_ck = __half2half2(__high2half(as_h2(cf.y)));
    const __half2 c_rp = __half2half2(__low2half(as_h2(cf.z)));
    const int sq = c.word & 63;
    const int ts = min(static_cast<int>(((c.word >> 6) & 7) * 2 + ((c.word >> 9) & 1)), kNTypeSpecial - 1);
    const int ct = (c.lane >> 4) * 2 + c.stm;
    const uint4* e_sq = reinterpret_cast<const uint4*>(p.emb + (EMB_SQUARE + sq) * kD + col);
    const uint4* e_ts = reinterpret_cast<const uint4*>(p.emb + (EMB_TS + ts) * kD + col);
    const uint4* e_ct = reinterpret_cast<const uint4*>(p.emb + (EMB_CT + ct) * kD + col);
    const uint4* e_ck = reinterpret_cast<const uint4*>(p.emb + (EMB_CLOCK + c.clk) * kD + col);
    const uint4* e_rp = reinterpret_cast<const uint4*>(p.emb + (EMB_REP + c.rp) * kD + col);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint4 a = __ldg(e_sq + k), b = __ldg(e_ts + k), d = __ldg(e_ct + k);
        const uint4 e = __ldg(e_ck + k), f = __ldg(e_rp + k);
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        const uint32_t dw[4] = {d.x, d.y, d.z, d.w}, ew[4] = {e.x, e.y, e.z, e.w};
        const uint32_t fw[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __half2 pb = __hfma2(c_ck, as_h2(ew[j]), __hmul2(c_rp, as_h2(fw[j])));
            const __half2 cs = __hfma2(c_ct, as_h2(dw[j]), pb);
            __half2 t = __hfma2(c_sq, as_h2(aw[j]), as_h2(x[4 * k + j]));
            t = __hfma2(c_ts, as_h2(bw[j]), t);
            x[4 * k + j] = as_u32(__hadd2(t, cs));
        }
    }
}

//
// In the e4m3 arithmetic the attention norm is not quantised at all: x_hat goes out as the fp16
// A operand of the fp16 QKV GEMM (`f16_out`); the FFN norm is quantised to e4m3 with scale
// amax/8 (csrc/fp8_gemm.cuh:147-208).  In the fp16 arithmetic both norms go out as fp16.
template <bool kDbg, bool kRJ, int kAr>
__device__ __forceinline__ float ln_stage(RowCtx& c, const Params& p, bool final_norm, bool dump_x,
                                          bool dump_xn, bool capture, int site, bool f16_out = false) {
    constexpr bool kFP8 = kAr == kArE4M3, kHalfA = kAr != kArInt8;
    // Partial sums in the reference's order (encoder.cu:566-583): "lane" l of the reference
    // owns columns 8l..8l+7 and adds them one after the other, then lanes combine by the
    // butterfly 16, 8, 4, 2, 1.  This thread's 64 columns are lanes 4qt..4qt+3 and their
    // partners 16 + 4qt..: it forms P[l] + P[l+16] for its four l (level 16); levels 8 and 4
    // pair it with the other three quarters of the row, levels 2 and 1 are local again.
    // Two lanes ride in one packed register: (x[l][j], x[l+1][j]).
    uint64_t as0 = 0, as1 = 0, aq0 = 0, aq1 = 0;
    __half2 mn = __float2half2_rn(65504.0f), mx = __float2half2_rn(-65504.0f);
    // both halves' loads are issued before the first is used: the second is in flight while
    // the first is summed
    uint32_t xa[16], xb2[16];
    tmem_ld16(c.tm + TM_X + 16 * c.qt, xa);
    tmem_wait_ld();
    tmem_ld16(c.tm + TM_X + 64 + 16 * c.qt, xb2);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        if (u == 1) tmem_wait_ld();
        uint32_t(&x)[16] = u ? xb2 : xa;
        if (kDbg && dump_x && c.valid) store_words<16>(p.y + c.grow * kD + 128 * u + 32 * c.qt, x);
        if (kRJ && site >= 0) reinject32(c, p, site, 128 * u + 32 * c.qt, x);
        uint64_t s2[2], q2[2];
#pragma unroll
        for (int pr = 0; pr < 2; ++pr) {
            s2[pr] = pk2(0.f, 0.f);
            q2[pr] = pk2(0.f, 0.f);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t wa = x[8 * pr + k], wb = x[8 * pr + 4 + k];
                uint64_t f = h2_to_f2(__byte_perm(wa, wb, 0x5410));
                s2[pr] = add2(s2[pr], f);
                q2[pr] = fma2(f, f, q2[pr]);
                f = h2_to_f2(__byte_perm(wa, wb, 0x7632));
                s2[pr] = add2(s2[pr], f);
                q2[pr] = fma2(f, f, q2[pr]);
            }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            mn = __hmin2(mn, as_h2(x[i]));
            mx = __hmax2(mx, as_h2(x[i]));
        }
        if (u == 0) {
            as0 = s2[0]; as1 = s2[1]; aq0 = q2[0]; aq1 = q2[1];
        } else {
            as0 = add2(as0, s2[0]); as1 = add2(as1, s2[1]);
            aq0 = add2(aq0, q2[0]); aq1 = add2(aq1, q2[1]);
        }
    }
    // Exchange among the row's four threads through this board's slice of the staging region
    // (idle between the MMAs that last read it and the next staging write): [sums | squares]
    // in the first 16 KB block,
    // [min, max] in the second.
    float tot, totq, xmin, xmax;
    {
        const uint32_t xb = c.sm_r + 4096u * c.q, slot = 16u * (32 * c.qt + c.lane);
        float f0, f1, f2, f3;
        upk2(as0, f0, f1); upk2(as1, f2, f3);
        sts_f4(xb + slot, make_float4(f0, f1, f2, f3));
        upk2(aq0, f0, f1); upk2(aq1, f2, f3);
        sts_f4(xb + 2048u + slot, make_float4(f0, f1, f2, f3));
        sts_f4(xb + 16384u + slot, make_float4(fminf(__low2float(mn), __high2float(mn)),
                                               fmaxf(__low2float(mx), __high2float(mx)), 0.f, 0.f));
        // the second pass's first half is fetched while the exchange is under way
        tmem_ld16(c.tm + TM_X + 16 * c.qt, xa);
        board_sync(c);
        float4 S[4], Q[4], M[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            S[k] = lds_f4(xb + 16u * (32 * k + c.lane));
            Q[k] = lds_f4(xb + 2048u + 16u * (32 * k + c.lane));
            M[k] = lds_f4(xb + 16384u + 16u * (32 * k + c.lane));
        }
        // The final norm writes its output over these slots right away, so every warp must have
        // read first.  After the other norms the next writer of this slice is an epilogue that
        // waits for a GEMM which itself waits for all sixteen warps' operand rows, written
        // after these reads: no second barrier is needed.
        if (final_norm) board_sync(c);
        // levels 8 and 4: (A_q0 + A_q2) + (A_q1 + A_q3) for each of the four lanes; level 2:
        // lanes (0,2) and (1,3); level 1: the last add
        const uint64_t c01 = add2(add2(pk2(S[0].x, S[0].y), pk2(S[2].x, S[2].y)),
                                  add2(pk2(S[1].x, S[1].y), pk2(S[3].x, S[3].y)));
        const uint64_t c23 = add2(add2(pk2(S[0].z, S[0].w), pk2(S[2].z, S[2].w)),
                                  add2(pk2(S[1].z, S[1].w), pk2(S[3].z, S[3].w)));
        const uint64_t d01 = add2(add2(pk2(Q[0].x, Q[0].y), pk2(Q[2].x, Q[2].y)),
                                  add2(pk2(Q[1].x, Q[1].y), pk2(Q[3].x, Q[3].y)));
        const uint64_t d23 = add2(add2(pk2(Q[0].z, Q[0].w), pk2(Q[2].z, Q[2].w)),
                                  add2(pk2(Q[1].z, Q[1].w), pk2(Q[3].z, Q[3].w)));
        float a, b;
        upk2(add2(c01, c23), a, b);
        tot = __fadd_rn(a, b);
        upk2(add2(d01, d23), a, b);
        totq = __fadd_rn(a, b);
        xmin = fminf(fminf(M[0].x, M[1].x), fminf(M[2].x, M[3].x));
        xmax = fmaxf(fmaxf(M[0].y, M[1].y), fmaxf(M[2].y, M[3].y));
    }
    const float mean = __fmul_rn(tot, 1.0f / 256.0f);
    // `sq / Dm - mean * mean` (encoder.cu:596): the product is rounded on its own, the
    // scaling by 1/256 is exact
    const float var = fmaxf(__fsub_rn(__fmul_rn(totq, 1.0f / 256.0f), __fmul_rn(mean, mean)), 0.f);
    const float rstd = p.rsqrt_rn ? __frsqrt_rn(__fadd_rn(var, p.eps)) : rsqrtf(__fadd_rn(var, p.eps));
    const float e_lo = __half2float(__float2half_rn(__fmul_rn(__fsub_rn(xmin, mean), rstd)));
    const float e_hi = __half2float(__float2half_rn(__fmul_rn(__fsub_rn(xmax, mean), rstd)));
    const float amax = fmaxf(fabsf(e_lo), fabsf(e_hi));
    const float sc = amax > 0.f ? __fdiv_rn(amax, kFP8 ? kQMaxE4M3 : kQMaxS8) : 1.0f;
    const float inv = __fdiv_rn(1.0f, sc);
    const uint64_t nmean2 = pk2(-mean, -mean), rstd2 = pk2(rstd, rstd);
    tmem_wait_ld();
    tmem_ld16(c.tm + TM_X + 64 + 16 * c.qt, xb2);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        if (u == 1) tmem_wait_ld();
        uint32_t(&x)[16] = u ? xb2 : xa;
        const int col = 128 * u + 32 * c.qt;
        if (kRJ && site >= 0) reinject32(c, p, site, col, x);
        if (!final_norm) {
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = f2_to_h2(mul2(add2(h2_to_f2(x[i]), nmean2), rstd2));
            if (kHalfA && f16_out) {
                // fp16 A operand: 4 K-slabs of [128 rows][64 halves]; this thread's 32 columns
                // are half of slab col / 64
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    sts128(c.sm_a + (2 * u + (c.qt >> 1)) * 16384 + sw_off(c.row, 4 * (c.qt & 1) + v),
                           make_uint4(x[4 * v], x[4 * v + 1], x[4 * v + 2], x[4 * v + 3]));
            } else {
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const uint4 qv = quant16_any<kFP8>(&x[8 * v], inv, c.one2);
                    sts128(c.sm_a + u * 16384 + sw_off(c.row, 2 * c.qt + v), qv);
                    if (kDbg && capture && c.valid) *reinterpret_cast<uint4*>(p.cap_a + c.grow * kD + col + 16 * v) = qv;
                }
            }
        } else {
            // norm_f with affine: fp16(fma(x_hat, gamma, beta)) (encoder.cu:609-611), written as
            // the fp16 A operand of the head product: 4 K-slabs of [128 rows][64 halves]
            const uint4* g4 = reinterpret_cast<const uint4*>(p.tail + col);
            const uint4* b4 = reinterpret_cast<const uint4*>(p.tail + kD + col);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 gv = __ldg(g4 + v), bv = __ldg(b4 + v);
                const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    x[4 * v + j] = f2_to_h2(fma2(mul2(add2(h2_to_f2(x[4 * v + j]), nmean2), rstd2),
                                                 h2_to_f2(gw[j]), h2_to_f2(bw[j])));
                // head A slab = col / 64 = 2u + qt/2; 16-byte group within the 64-column slab
                sts128(c.sm_r + (2 * u + (c.qt >> 1)) * 16384 + sw_off(c.row, 4 * (c.qt & 1) + v),
                       make_uint4(x[4 * v], x[4 * v + 1], x[4 * v + 2], x[4 * v + 3]));
            }
        }
        if (kDbg && dump_xn && c.valid) store_words<16>(p.y + c.grow * kD + col, x);
    }
    return sc;
}

// Half of one (board, head) attention unit: 16 query rows against the board's 32 keys, on the
// staged fp16 Q/K/V of a head pair, instruction for instruction what the reference does
// (encoder.cu:715-797): S = Q K^T (scale pre-folded) on m16n8k16 with fp16 accumulators, dims
// 0-15 before 16-31; dead keys -inf; row max; __expf(s - max); the row sum in the reference's
// order; P = fp16(p * (1 / sum)); O = P V on the same instruction, keys 0-15 before 16-31.  Warp (q, qt) takes head
// qt & 1 of the pair and query rows 16 * (qt >> 1) .. +15; the result overwrites its own
// block of Q.
__device__ __forceinline__ void attention_unit(const RowCtx& c, uint32_t alive) {
    const uint32_t qs = c.sm_r, ks = qs + 16384, vs = qs + 32768;
    const int hh = c.qt & 1, r0 = 32 * c.q, rq = r0 + 16 * (c.qt >> 1);
    const int lane = c.lane, g = lane >> 2, t = lane & 3;
    uint32_t qa[2][4];
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
        const int row = rq + (lane & 15);
        ldmatrix_x4(qa[kk], qs + sw_off(row, 4 * hh + 2 * kk + (lane >> 4)));
    }
    // s[nt] = {row g, row g + 8} x key columns 8 nt + 2t, +1, as packed fp16 pairs
    uint32_t s[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        s[nt][0] = s[nt][1] = 0u;
        uint32_t kb[4];
        const int row = r0 + 8 * nt + (lane & 7);
        ldmatrix_x4(kb, ks + sw_off(row, 4 * hh + (lane >> 3)));
        mma_f16_f16(s[nt], qa[0], kb[0], kb[1]);      // dims 0-15, then 16-31
        mma_f16_f16(s[nt], qa[1], kb[2], kb[3]);
    }
    // dead keys -> -inf: this lane's two keys of every n-tile are the same for both row halves,
    // so the mask is one packed fp16 pair per n-tile (0 keeps a score bit for bit, -inf replaces
    // it: a finite fp16 plus -inf is -inf) and applying it is one packed add per pair
    uint32_t dead[4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const uint32_t two = (alive >> (8 * nt + 2 * t)) & 3u;
        dead[nt] = ((two & 1u) ? 0u : 0xfc00u) | ((two & 2u) ? 0u : 0xfc000000u);
    }
#pragma unroll
    for (int hi = 0; hi < 2; ++hi) {
        float pv[4][2];
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const __half2 val = __hadd2(as_h2(s[nt][hi]), as_h2(dead[nt]));
            pv[nt][0] = __low2float(val);
            pv[nt][1] = __high2float(val);
            mx = fmaxf(mx, fmaxf(pv[nt][0], pv[nt][1]));
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        float sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            pv[nt][0] = __expf(pv[nt][0] - mx);       // an all-dead row keeps the reference's NaN
            pv[nt][1] = __expf(pv[nt][1] - mx);
            sum += pv[nt][0] + pv[nt][1];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        const float inv = 1.0f / sum;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) s[nt][hi] = pack_h2(pv[nt][0] * inv, pv[nt][1] * inv);
    }
    // P's accumulator fragments are already A fragments: keys 16 kk .. +15 are n-tiles 2kk, 2kk+1
    uint32_t pa[2][4];
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
        pa[kk][0] = s[2 * kk][0];     pa[kk][1] = s[2 * kk][1];
        pa[kk][2] = s[2 * kk + 1][0]; pa[kk][3] = s[2 * kk + 1][1];
    }
    uint32_t o[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        o[nt][0] = o[nt][1] = 0u;
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vs + sw_off(r0 + lane, 4 * hh + nt));
        mma_f16_f16(o[nt], pa[0], vb[0], vb[1]);      // keys 0-15, then 16-31
        mma_f16_f16(o[nt], pa[1], vb[2], vb[3]);
    }
    // the outputs go to the staging region's fourth block, which nothing else uses during the
    // attention loop: the next head pair's Q, K and V can then be staged while a slower warp of
    // the board is still reading these back
    const uint32_t os = qs + 49152;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
        const int row = rq + g;
        sts32(os + sw_off(row, 4 * hh + nt) + 4 * t, o[nt][0]);
        sts32(os + sw_off(row + 8, 4 * hh + nt) + 4 * t, o[nt][1]);
    }
}

// ------------------------------------------------------------------------------------------
// Row-warp work, written as run-time loops over column groups so that the whole layer body
// stays small enough for the instruction cache.
// ------------------------------------------------------------------------------------------
struct LayerParams {
    const float *sw_qkv, *sw_o, *sw_ff1, *sw_ff2;
    const __half *b_qkv, *b_o, *b_ff1, *b_ff2;
};

// QKV in four head-pair chunks with attention per chunk, then the attention output is
// quantised into A, then out-projection + residual into the residual stream (TMEM).
// `sa` is the scale of the row in A on entry.
template <bool kDbg, int kAr>
__device__ __forceinline__ void attention_block(RowCtx& c, const Params& p, const LayerParams& lp,
                                                float sa, uint32_t alive, bool cap, bool dbgl) {
    constexpr bool kHalfA = kAr != kArInt8;
    const int dbg = p.debug_stage;
    float o_amax = 0.f;
#pragma unroll 1
    for (int j = 0; j < 4; ++j) {
        row_wait_acc<kDbg>(c, 0, j == 0 ? PH_LN : PH_PAIR_BAR);
        // this thread's 48 of the chunk's 192 columns, 16 at a time; the load of the next group
        // is in flight while a group is descaled and staged
        {
            uint32_t pa[16], pb[16];
            tmem_ld16(c.tm + TM_ACC + 48 * c.qt, pa);
            tmem_wait_ld();
#pragma unroll
            for (int g = 0; g < 3; ++g) {
                uint32_t* cur = (g & 1) ? pb : pa;
                uint32_t* nxt = (g & 1) ? pa : pb;
                if (g < 2) tmem_ld16(c.tm + TM_ACC + 48 * c.qt + 16 * (g + 1), *reinterpret_cast<uint32_t(*)[16]>(nxt));
                const int c0 = 48 * c.qt + 16 * g, m = c0 >> 6, cm = c0 & 63;
                uint32_t h[8];
                if (kDbg && cap && p.cap_op == BF_OP_QKV && c.valid)
                    store_words<16>(p.cap_acc + c.grow * 768 + j * 192 + c0, cur);
                descale<16, false, Cfg<kAr>::kQkvF16 ? kAccPlain : kAccInt>(cur, sa, __ldg(lp.sw_qkv + m * 2 + (j >> 1)),
                                                                lp.b_qkv + j * 192 + c0, h);
#pragma unroll
                for (int k = 0; k < 2; ++k)
                    sts128(c.sm_r + m * 16384 + sw_off(c.row, (cm >> 3) + k),
                           make_uint4(h[4 * k], h[4 * k + 1], h[4 * k + 2], h[4 * k + 3]));
                if (kDbg && dbgl && dbg == 5 + m && c.valid) store_words<8>(p.y + c.grow * kD + 64 * j + cm, h);
                if (g < 2) tmem_wait_ld();
            }
        }
        row_release_acc(c, 0);
        prof_mark<kDbg>(c, PH_QKV_EPI);
        board_sync(c);                     // this board's Q/K/V rows are staged
        prof_mark<kDbg>(c, PH_PAIR_BAR);
        attention_unit(c, alive);
        prof_mark<kDbg>(c, PH_ATTENTION);
        board_sync(c);                     // all four warps' outputs are in the output block
        {
            // read back 16 of this row's 64 outputs of the head pair, park them in tensor memory
            uint32_t oh[8];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const uint4 v = lds128(c.sm_r + 49152 + sw_off(c.row, 2 * c.qt + k));
                oh[4 * k] = v.x; oh[4 * k + 1] = v.y; oh[4 * k + 2] = v.z; oh[4 * k + 3] = v.w;
            }
            o_amax = fmaxf(o_amax, amax_h2<8>(oh, true));
            tmem_st8(c.tm + TM_OY + 32 * j + 8 * c.qt, oh);
            if (kDbg && dbgl && dbg == 4 && c.valid) store_words<8>(p.y + c.grow * kD + 64 * j + 16 * c.qt, oh);
        }
        prof_mark<kDbg>(c, PH_O_READBACK);
        // no barrier here: the next head pair's staging does not touch the output block, and its
        // attention units (which do) start only after the barrier that follows that staging,
        // which every warp reaches after this read-back
    }
    tmem_wait_st();
    prof_mark<kDbg>(c, PH_PAIR_BAR);

    // the attention output becomes the A operand of the out-projection: quantised to s8 with a
    // per-row scale, or (e4m3 and fp16 arithmetics) copied as fp16 into the four fp16 K-slabs
    if (kHalfA) {
#pragma unroll 1
        for (int j = 0; j < 4; ++j) {
            uint32_t oh[8];
            tmem_ld8(c.tm + TM_OY + 32 * j + 8 * c.qt, oh);
            tmem_wait_ld();
            // columns 64j + 16qt .. +15 of the fp16 operand: slab j, 16-byte groups 2qt, 2qt+1
            sts128(c.sm_a + j * 16384 + sw_off(c.row, 2 * c.qt), make_uint4(oh[0], oh[1], oh[2], oh[3]));
            sts128(c.sm_a + j * 16384 + sw_off(c.row, 2 * c.qt + 1), make_uint4(oh[4], oh[5], oh[6], oh[7]));
        }
        row_publish(c, B_A_READY);
    } else {
        // the four pieces' loads go out together, ahead of the row maximum's exchange
        uint32_t oh[4][8];
#pragma unroll
        for (int j = 0; j < 4; ++j) tmem_ld8(c.tm + TM_OY + 32 * j + 8 * c.qt, oh[j]);
        const float amax = exchange_max(c, o_amax);
        sa = amax > 0.f ? __fdiv_rn(amax, kQMaxS8) : 1.0f;
        const float inv = __fdiv_rn(1.0f, sa);
        const bool capo = kDbg && cap && p.cap_op == BF_OP_OUT && c.valid;
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint4 v = quant16(oh[j], inv, c.one2);
            sts128(c.sm_a + (j >> 1) * 16384 + sw_off(c.row, 4 * (j & 1) + c.qt), v);
            if (capo) *reinterpret_cast<uint4*>(p.cap_a + c.grow * kD + 64 * j + 16 * c.qt) = v;
        }
        row_publish(c, B_A_READY);
    }

    // out-projection: x = fp16(x + fp16(fp16(descale) + b_o)) (encoder.cu:631-686)
#pragma unroll 1
    for (int u = 0; u < 2; ++u) {
        row_wait_acc<kDbg>(c, u, u == 0 ? PH_O_QUANT : PH_OUT_EPI, PH_WAIT_OUT);
        const int col = 128 * u + 32 * c.qt;
        uint32_t acc[32], y[16], xo[16];
        tmem_ld32(c.tm + TM_ACC + col, acc);
        tmem_ld16(c.tm + TM_X + (col >> 1), xo);
        tmem_wait_ld();
        row_release_acc(c, u);
        if (kDbg && cap && p.cap_op == BF_OP_OUT && c.valid) store_words<32>(p.cap_acc + c.grow * 256 + col, acc);
        descale<32, false, Cfg<kAr>::kOutF16 ? kAccPlain : kAccInt>(acc, sa, __ldg(lp.sw_o + u), lp.b_o + col, y);
#pragma unroll
        for (int i = 0; i < 16; ++i) xo[i] = as_u32(__hadd2(as_h2(xo[i]), as_h2(y[i])));
        tmem_st16(c.tm + TM_X + (col >> 1), xo);
    }
    tmem_wait_st();
    prof_mark<kDbg>(c, PH_OUT_EPI);
}

// FFN: four hidden chunks of 256; ff1 -> ReLU -> per-row u8 -> ff2 with an fp16 running
// total (encoder.cu:1431-1556).  The eight steps follow the MMA issue order.
template <bool kDbg, int kAr>
__device__ __forceinline__ void ffn_block(RowCtx& c, const Params& p, const LayerParams& lp,
                                          float sa, bool cap) {
    constexpr bool kFP8 = kAr == kArE4M3;
    static_assert(kAr != kArF16, "the fp16 arithmetic has its own FFN block");
    float sa2_0 = 1.f, sa2_1 = 1.f;
    prof_mark<kDbg>(c, PH_LN);
#pragma unroll 1
    for (int st = 0; st < 8; ++st) {
        const int kind2 = (0xD4 >> st) & 1;
        const int ch = kind2 ? ((0x32010000u >> (4 * st)) & 0xF) : ((0x00302010u >> (4 * st)) & 0xF);
        if (!kind2) {
            // 64 columns in four 16-column pieces (two per accumulator slot); the tensor-memory
            // load of a piece is in flight while the piece before it is descaled
            uint32_t hid[32];
            {
                constexpr int kA = kFP8 ? kAccFloat : kAccInt;
                const bool capf = kDbg && cap && p.cap_op == BF_OP_FF1 && c.valid;
                const int col0 = 256 * ch + 32 * c.qt;                 // + 128 jh + 16 half
                const uint32_t t0 = c.tm + TM_ACC + 32 * c.qt;
                const float sw0 = __ldg(lp.sw_ff1 + 2 * ch), sw1 = __ldg(lp.sw_ff1 + 2 * ch + 1);
                uint32_t pa[16], pb[16];
                row_wait_acc<kDbg>(c, 0, PH_FF1_EPI, ch == 0 ? PH_WAIT_FF1_FIRST : PH_WAIT_FF1);
                tmem_ld16(t0, pa);
                tmem_wait_ld();
                tmem_ld16(t0 + 16, pb);
                if (capf) store_words<16>(p.cap_acc + c.grow * 1024 + col0, pa);
                descale<16, true, kA>(pa, sa, sw0, lp.b_ff1 + col0, &hid[0]);
                row_release_acc(c, 0);                                 // waits for the load of pb
                row_wait_acc<kDbg>(c, 1, PH_FF1_EPI, PH_WAIT_FF1);
                tmem_ld16(t0 + 128, pa);
                if (capf) store_words<16>(p.cap_acc + c.grow * 1024 + col0 + 16, pb);
                descale<16, true, kA>(pb, sa, sw0, lp.b_ff1 + col0 + 16, &hid[8]);
                tmem_wait_ld();
                tmem_ld16(t0 + 128 + 16, pb);
                if (capf) store_words<16>(p.cap_acc + c.grow * 1024 + col0 + 128, pa);
                descale<16, true, kA>(pa, sa, sw1, lp.b_ff1 + col0 + 128, &hid[16]);
                row_release_acc(c, 1);
                if (capf) store_words<16>(p.cap_acc + c.grow * 1024 + col0 + 144, pb);
                descale<16, true, kA>(pb, sa, sw1, lp.b_ff1 + col0 + 144, &hid[24]);
            }
            // per-row u8 scale over the 256-wide chunk (encoder.cu:1510-1517)
            const float amax = exchange_max(c, amax_h2<32>(hid, false));
            const float sc = amax > 0.f ? __fdiv_rn(amax, kFP8 ? kQMaxE4M3 : kQMaxU8) : 1.0f;
            const float inv = __fdiv_rn(1.0f, sc);
            if (ch & 1) sa2_1 = sc; else sa2_0 = sc;
            const bool caph = kDbg && cap && p.cap_op == BF_OP_FF2 + ch && c.valid;
#pragma unroll
            for (int jh = 0; jh < 2; ++jh)
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const uint4 v = quant16_any<kFP8>(&hid[16 * jh + 8 * k], inv, c.one2);
                    sts128(c.sm_r + (ch & 1) * 32768 + jh * 16384 + sw_off(c.row, 2 * c.qt + k), v);
                    if (caph) *reinterpret_cast<uint4*>(p.cap_a + c.grow * kD + 128 * jh + 32 * c.qt + 16 * k) = v;
                }
            row_publish(c, B_A2_READY + (ch & 1));
            prof_mark<kDbg>(c, PH_FF1_EPI);
        } else {
            const float s1 = (ch & 1) ? sa2_1 : sa2_0;
#pragma unroll 1
            for (int jh = 0; jh < 2; ++jh) {
                row_wait_acc<kDbg>(c, jh, PH_FF2_EPI, PH_WAIT_FF2);
                const float s2 = __ldg(lp.sw_ff2 + jh);
                // 32 columns as two 16-column pieces: the second piece's loads are in flight
                // while the first is accumulated
                uint32_t pa[16], pb[16], run[16];
                const int col = 128 * jh + 32 * c.qt;
                const bool capf = kDbg && cap && p.cap_op == BF_OP_FF2 + ch && c.valid;
                const uint64_t s1_2 = pk2(s1, s1), s2_2 = pk2(s2, s2);
                tmem_ld16(c.tm + TM_ACC + col, pa);
                if (ch > 0) tmem_ld8(c.tm + TM_OY + (col >> 1), *reinterpret_cast<uint32_t(*)[8]>(&run[0]));
                tmem_wait_ld();
                tmem_ld16(c.tm + TM_ACC + col + 16, pb);
                if (ch > 0) tmem_ld8(c.tm + TM_OY + (col >> 1) + 8, *reinterpret_cast<uint32_t(*)[8]>(&run[8]));
                if (capf) store_words<16>(p.cap_acc + c.grow * 256 + col, pa);
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    if (half == 1) {
                        row_release_acc(c, jh);                        // waits for the second piece
                        if (capf) store_words<16>(p.cap_acc + c.grow * 256 + col + 16, pb);
                    }
                    const uint32_t* acc = half ? pb : pa;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        uint64_t f = kFP8 ? pk2(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1]))
                                          : pk2(static_cast<float>(static_cast<int>(acc[2 * i])),
                                                static_cast<float>(static_cast<int>(acc[2 * i + 1])));
                        // `float(acc) * sa * sw + float(run)` (int8_gemm.cuh:285-294): the compiler
                        // fuses the second product with the sum in the reference, so it is one fma here
                        f = mul2(f, s1_2);
                        f = ch > 0 ? fma2(f, s2_2, h2_to_f2(run[8 * half + i])) : mul2(f, s2_2);
                        run[8 * half + i] = f2_to_h2(f);
                    }
                }
                if (ch < 3) {
                    tmem_st16(c.tm + TM_OY + (col >> 1), run);
                } else {
                    // + b_ff2, residual (encoder.cu:1548-1556): x = fp16(x + fp16(run + b))
                    uint32_t xo[16];
                    tmem_ld16(c.tm + TM_X + (col >> 1), xo);
                    tmem_wait_ld();
                    const uint4* b4 = reinterpret_cast<const uint4*>(lp.b_ff2 + col);
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const uint4 bv = __ldg(b4 + v);
                        const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int i = 4 * v + k;
                            const __half2 yv = __hadd2(as_h2(run[i]), as_h2(bw[k]));
                            xo[i] = as_u32(__hadd2(as_h2(xo[i]), yv));
                        }
                    }
                    tmem_st16(c.tm + TM_X + (col >> 1), xo);
                }
            }
            tmem_wait_st();
            prof_mark<kDbg>(c, PH_FF2_EPI);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Fused expansion: the node's legal edges and their priors straight from the staged logits,
// what the reference's search does in a kernel of its own after reading the logits back
// (Search._expand, brokefish/search/torch_impl.py:962-1033; csrc/search.cuh:593-798).  One warp
// per board, lane = piece slot.  A candidate is a legal (slot, square), four times over
// (N B R Q) when a pawn reaches its last rank; its logit is the policy logit plus, for a
// promotion, log_softmax of the slot's promotion logits, evaluated as (x - max) - log(sum);
// the prior is exp(logit - max) / sum over the kept candidates, stored as fp16.  More than
// `e_cap` candidates: the e_cap largest logits stay, ties to the earlier candidate.  Edges are
// written in canonical order (slot, square, type) whatever their prior.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t order_key(float v) {
    // unsigned keys that sort like the floats; -0 and +0 share a key
    uint32_t b = __float_as_uint(v);
    if (b == 0x80000000u) b = 0u;
    return (b & 0x80000000u) ? ~b : (b ^ 0x80000000u);
}
template <typename F>
__device__ __forceinline__ void each_candidate(unsigned long long legal, unsigned long long promos,
                                               uint32_t row_smem, uint32_t row_xor, const float (&type_lp)[4],
                                               F&& visit) {
    for (unsigned long long rest = legal; rest != 0ull; rest &= rest - 1ull) {
        const int sq = __ffsll(static_cast<long long>(rest)) - 1;
        uint16_t raw;
        asm volatile("ld.shared.u16 %0, [%1];"
                     : "=h"(raw)
                     : "r"(row_smem + (((static_cast<uint32_t>(sq) >> 3) ^ row_xor) << 4) + 2u * (sq & 7)));
        const float base = __half2float(__ushort_as_half(raw));
        if ((promos >> sq) & 1ull) {
#pragma unroll
            for (int t = 0; t < 4; ++t) visit(sq, t, __fadd_rn(base, type_lp[t]));
        } else {
            visit(sq, 0, base);
        }
    }
}
__device__ __forceinline__ int warp_prefix(int mine, int lane, int& total) {
    int inc = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= off) inc += up;
    }
    total = __shfl_sync(0xffffffffu, inc, 31);
    return inc - mine;
}
__device__ __forceinline__ float warp_sum_to_all(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_down_sync(0xffffffffu, v, off));
    return __shfl_sync(0xffffffffu, v, 0);
}
__device__ __forceinline__ void expand_board(const Params& p, int board, int lane, bool valid, uint32_t word,
                                             int ctl, unsigned long long legal, uint32_t stage_pol,
                                             uint32_t stage_aux, int row, uint8_t* list_buf) {
    // the staged row of this slot: 16-byte group g of the row lives at sw_off(row, g)
    const uint32_t row_smem = stage_pol + static_cast<uint32_t>(row) * 128u;
    const uint32_t row_xor = static_cast<uint32_t>(row & 7);
    const bool pawn = ((word >> 11) & 1u) == 0u && ((word >> 6) & 7u) == 0u;
    const unsigned long long last = ctl < 0 ? 0xffull : (0xffull << 56);
    const unsigned long long promos = pawn ? (legal & last) : 0ull;
    float type_lp[4] = {0.f, 0.f, 0.f, 0.f};
    if (promos != 0ull) {
        uint32_t w0, w1;
        asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(w0), "=r"(w1) : "r"(stage_aux + sw_off(row, 0)));
        const float x[4] = {__low2float(as_h2(w0)), __high2float(as_h2(w0)), __low2float(as_h2(w1)),
                            __high2float(as_h2(w1))};
        const float top = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
        float z = 0.f;
#pragma unroll
        for (int t = 0; t < 4; ++t) z = __fadd_rn(z, expf(__fsub_rn(x[t], top)));
        const float lz = logf(z);
#pragma unroll
        for (int t = 0; t < 4; ++t) type_lp[t] = __fsub_rn(__fsub_rn(x[t], top), lz);
    }
    const int e_cap = p.e_cap;
    int total = 0;
    const int mine = __popcll(legal) + 3 * __popcll(promos);
    int first = warp_prefix(mine, lane, total);          // this slot's first edge index
    // threshold of a truncating node: the e_cap-th largest key, found bit by bit
    const bool cut = total > e_cap;
    uint32_t thr = 0u;
    int ties_wanted = 0, tie_rank0 = 0;
    if (cut) {
#pragma unroll 1
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t trial = thr | (1u << bit);
            int at_least = 0;
            each_candidate(legal, promos, row_smem, row_xor, type_lp, [&](int, int, float lg) { at_least += order_key(lg) >= trial; });
            if (__reduce_add_sync(0xffffffffu, static_cast<unsigned>(at_least)) >= static_cast<unsigned>(e_cap)) thr = trial;
        }
        int above = 0, equal = 0;
        each_candidate(legal, promos, row_smem, row_xor, type_lp, [&](int, int, float lg) {
            const uint32_t k = order_key(lg);
            above += k > thr;
            equal += k == thr;
        });
        int above_all = 0, equal_all = 0;
        const int above_before = warp_prefix(above, lane, above_all);
        tie_rank0 = warp_prefix(equal, lane, equal_all);
        ties_wanted = e_cap - above_all;
        first = above_before + min(tie_rank0, ties_wanted);
    }
    // a candidate stays when it beats the threshold, or ties with it early enough
    int tie_rank = tie_rank0;
    auto stays = [&](float lg) -> bool {
        if (!cut) return true;
        const uint32_t k = order_key(lg);
        if (k > thr) return true;
        if (k < thr) return false;
        return tie_rank++ < ties_wanted;
    };
    float top = -INFINITY;
    each_candidate(legal, promos, row_smem, row_xor, type_lp, [&](int, int, float lg) { if (stays(lg)) top = fmaxf(top, lg); });
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
    tie_rank = tie_rank0;
    float part = 0.f;
    each_candidate(legal, promos, row_smem, row_xor, type_lp, [&](int, int, float lg) {
        if (stays(lg)) part = __fadd_rn(part, expf(__fsub_rn(lg, top)));
    });
    const float z = warp_sum_to_all(part);
    const int kept = cut ? e_cap : total;
    if (valid) {
        // The edge list is put together in shared memory (`list_buf`: 1 KB, priors in the first
        // half, labels in the second) and leaves in 16-byte stores: the outputs may be pinned host
        // memory, where every store is a transaction on the bus.
        __half* out_p = p.prior + static_cast<size_t>(board) * e_cap;
        int16_t* out_m = p.move + static_cast<size_t>(board) * e_cap;
        __half* list_p = reinterpret_cast<__half*>(list_buf);
        int16_t* list_m = reinterpret_cast<int16_t*>(list_buf + 512);
        tie_rank = tie_rank0;
        int at = first;
        each_candidate(legal, promos, row_smem, row_xor, type_lp, [&](int sq, int t, float lg) {
            if (!stays(lg)) return;
            list_p[at] = __float2half_rn(__fdiv_rn(expf(__fsub_rn(lg, top)), z));
            list_m[at] = static_cast<int16_t>((lane * 64 + sq) | (t << 11));
            ++at;
        });
        for (int i = kept + lane; i < e_cap; i += 32) { list_p[i] = __float2half_rn(0.f); list_m[i] = 0; }
        __syncwarp();
        const bool wide = (e_cap & 7) == 0 &&
                          ((reinterpret_cast<uintptr_t>(out_p) | reinterpret_cast<uintptr_t>(out_m)) & 15u) == 0;
        if (wide) {
            for (int i = lane; i < e_cap / 8; i += 32) {
                reinterpret_cast<uint4*>(out_p)[i] = reinterpret_cast<const uint4*>(list_p)[i];
                reinterpret_cast<uint4*>(out_m)[i] = reinterpret_cast<const uint4*>(list_m)[i];
            }
        } else {
            for (int i = lane; i < e_cap; i += 32) { out_p[i] = list_p[i]; out_m[i] = list_m[i]; }
        }
        if (lane == 0) p.nedges[board] = kept;
    }
}

// FFN of the fp16 arithmetic (the reference's default path, csrc/encoder.cu:1431-1556 with
// Q8 = false): ff1 per 256-wide hidden chunk as an fp16 GEMM with fp16 accumulators, + bias, ReLU
// in fp16; the chunk goes out as the fp16 A operand of ff2, whose fp16 accumulators run on
// through all four chunks (K = 1024 in 64 steps of 16) before bias and residual are added.
// One hidden buffer (the whole 64 KB staging region): a chunk may be written only when the ff2
// units of the chunk before it have completed, which the MMA issuer signals on accumulator
// barrier 1 once per chunk.  ff1 units use accumulator slot 0; the ff2 accumulators are the
// (idle) attention-output columns for output half 0 and slot 1 for half 1.
template <bool kDbg>
__device__ __forceinline__ void ffn_block_f16(RowCtx& c, const Params& p, const LayerParams& lp) {
    prof_mark<kDbg>(c, PH_LN);
#pragma unroll 1
    for (int ch = 0; ch < 4; ++ch) {
#pragma unroll 1
        for (int jh = 0; jh < 2; ++jh) {
            row_wait_acc<kDbg>(c, 0, PH_FF1_EPI, ch == 0 && jh == 0 ? PH_WAIT_FF1_FIRST : PH_WAIT_FF1);
            uint32_t acc[32], hid[16];
            tmem_ld32(c.tm + TM_ACC + 32 * c.qt, acc);
            tmem_wait_ld();
            row_release_acc(c, 0);
            descale<32, true, kAccPlain>(acc, 1.f, 1.f, lp.b_ff1 + 256 * ch + 128 * jh + 32 * c.qt, hid);
            // the ff2 units of the previous chunk must be done with the hidden buffer
            if (ch > 0 && jh == 0) row_wait_acc<kDbg>(c, 1, PH_FF1_EPI, PH_WAIT_FF2);
            // columns 128 jh + 32 qt .. +31 of the chunk: K-slab 2 jh + qt / 2, 16-byte groups
            // 4 (qt & 1) .. +3
#pragma unroll
            for (int v = 0; v < 4; ++v)
                sts128(c.sm_r + (2 * jh + (c.qt >> 1)) * 16384 + sw_off(c.row, 4 * (c.qt & 1) + v),
                       make_uint4(hid[4 * v], hid[4 * v + 1], hid[4 * v + 2], hid[4 * v + 3]));
        }
        row_publish(c, B_A2_READY);
        prof_mark<kDbg>(c, PH_FF1_EPI);
    }
    // all four chunks accumulated: + b_ff2, residual (encoder.cu:1548-1556)
    row_wait_acc<kDbg>(c, 1, PH_FF1_EPI, PH_WAIT_FF2);
#pragma unroll 1
    for (int jh = 0; jh < 2; ++jh) {
        uint32_t acc[32], y[16], xo[16];
        const int col = 128 * jh + 32 * c.qt;
        tmem_ld32(c.tm + (jh ? TM_ACC + 128 : TM_OY) + 32 * c.qt, acc);
        tmem_ld16(c.tm + TM_X + (col >> 1), xo);
        tmem_wait_ld();
        descale<32, false, kAccPlain>(acc, 1.f, 1.f, lp.b_ff2 + col, y);
#pragma unroll
        for (int i = 0; i < 16; ++i) xo[i] = as_u32(__hadd2(as_h2(xo[i]), as_h2(y[i])));
        tmem_st16(c.tm + TM_X + (col >> 1), xo);
    }
    row_release_acc(c, 1);
    tmem_wait_st();
    prof_mark<kDbg>(c, PH_FF2_EPI);
}

// The "prenorm" value head (csrc/encoder.cu:1008-1057; nn/model.py:576-584): the raw residual
// stream is averaged over the board's live tokens, that one vector goes through the final
// LayerNorm (with affine) and is dotted with the value rows, all in fp32.  Written as one pass
// over this thread's 64 columns: with a = the column means, the k-th logit is
// rstd * (sum a*g*w_k - mean * sum g*w_k) + sum b*w_k, so no vector has to be kept.
// Every thread of the board returns the same three logits.
__device__ __forceinline__ void prenorm_value(RowCtx& c, const Params& p, uint32_t alive, float (&logit)[3]) {
    const bool live = (alive >> c.lane) & 1u;
    const int nlive = __popc(alive);
    const float inv_live = 1.0f / static_cast<float>(nlive > 0 ? nlive : 1);
    float s = 0.f, q = 0.f, s1[3] = {0.f, 0.f, 0.f}, s2[3] = {0.f, 0.f, 0.f}, s3[3] = {0.f, 0.f, 0.f};
#pragma unroll 1
    for (int u = 0; u < 2; ++u) {
        uint32_t x[16];
        tmem_ld16(c.tm + TM_X + 64 * u + 16 * c.qt, x);
        tmem_wait_ld();
        const int col = 128 * u + 32 * c.qt;
#pragma unroll 1
        for (int i = 0; i < 16; ++i) {
            const float2 f = __half22float2(as_h2(x[i]));
            float a0 = live ? f.x : 0.f, a1 = live ? f.y : 0.f;
#pragma unroll
            for (int off = 16; off; off >>= 1) {
                a0 += __shfl_xor_sync(0xffffffffu, a0, off);
                a1 += __shfl_xor_sync(0xffffffffu, a1, off);
            }
            a0 *= inv_live; a1 *= inv_live;
            s += a0 + a1;
            q += a0 * a0 + a1 * a1;
            const float2 g = __half22float2(as_h2(__ldg(reinterpret_cast<const uint32_t*>(p.tail + col) + i)));
            const float2 b = __half22float2(as_h2(__ldg(reinterpret_cast<const uint32_t*>(p.tail + kD + col) + i)));
#pragma unroll
            for (int k = 0; k < 3; ++k) {
                const float2 w = __half22float2(
                    as_h2(__ldg(reinterpret_cast<const uint32_t*>(p.tail + 2 * kD + k * kD + col) + i)));
                s1[k] += a0 * g.x * w.x + a1 * g.y * w.y;
                s2[k] += g.x * w.x + g.y * w.y;
                s3[k] += b.x * w.x + b.y * w.y;
            }
        }
    }
    float4 all[4];
    exchange4(c, make_float4(s, q, 0.f, 0.f), all);
    const float tot = (all[0].x + all[1].x) + (all[2].x + all[3].x);
    const float totq = (all[0].y + all[1].y) + (all[2].y + all[3].y);
    const float mean = tot * (1.0f / 256.0f);
    const float rstd = rsqrtf(fmaxf(__fsub_rn(totq * (1.0f / 256.0f), __fmul_rn(mean, mean)), 0.f) + p.eps);
    float t1[3], t2[3], t3[3];
    exchange4(c, make_float4(s1[0], s1[1], s1[2], 0.f), all);
    t1[0] = (all[0].x + all[1].x) + (all[2].x + all[3].x);
    t1[1] = (all[0].y + all[1].y) + (all[2].y + all[3].y);
    t1[2] = (all[0].z + all[1].z) + (all[2].z + all[3].z);
    exchange4(c, make_float4(s2[0], s2[1], s2[2], 0.f), all);
    t2[0] = (all[0].x + all[1].x) + (all[2].x + all[3].x);
    t2[1] = (all[0].y + all[1].y) + (all[2].y + all[3].y);
    t2[2] = (all[0].z + all[1].z) + (all[2].z + all[3].z);
    exchange4(c, make_float4(s3[0], s3[1], s3[2], 0.f), all);
    t3[0] = (all[0].x + all[1].x) + (all[2].x + all[3].x);
    t3[1] = (all[0].y + all[1].y) + (all[2].y + all[3].y);
    t3[2] = (all[0].z + all[1].z) + (all[2].z + all[3].z);
#pragma unroll
    for (int k = 0; k < 3; ++k) logit[k] = rstd * (t1[k] - mean * t2[k]) + t3[k];
}

// The head epilogue of one board: accumulators of the head product -> staged logits -> legality
// mask, stores, fused expansion, value.
template <bool kDbg>
__device__ __forceinline__ void head_epilogue(RowCtx& c, const Params& p, int board, uint32_t word, int ctl,
                                              uint32_t alive) {
    // ---- heads: fp16 product [128 x 256] x [96 x 256]^T on the tensor pipe (tcgen05 kind::f16
    //      with fp16 accumulators, k-steps in rising order: the bits of the reference's
    //      fp16-accumulate mma.sync product, encoder.cu:309-352, 918-927).  Warp qt of a board
    //      reads its rows' output columns 24 qt .. 24 qt + 23; they go through a staging tile in
    //      the (idle) A-operand region so that each thread then finds its own row's 16 policy
    //      columns and the expansion warp whole rows. ----
    float pre[3] = {0.f, 0.f, 0.f};
    if (p.vmode == 2) prenorm_value(c, p, c.valid ? alive : 0xffffffffu, pre);
    prof_mark<kDbg>(c, PH_LN);
    // Staging uses only this board's own rows of the A-operand slabs (another board may already
    // be writing its rows for the next tile): policy columns 0-63 in K-slab 0 at the operand's
    // swizzled row address, the 32 aux columns in K-slab 1.
    const uint32_t stage_pol = c.sm_a, stage_aux = c.sm_a + 16384u;
    // while the head product runs: the legality words, given or (for the expansion warp, lane =
    // slot) generated here
    unsigned long long lw = ~0ull, moves = 0ull;
    if (p.legal != nullptr && c.valid) lw = p.legal[c.grow];
    if (p.prior != nullptr && c.qt == 1 && c.valid) {
        bool in_check;
        moves = p.legal != nullptr ? lw : bfmg::legal_word(word, ctl, in_check);
    }
    row_wait_acc<kDbg>(c, 0, PH_LN);
    {
        // this thread's row, output columns 24 qt .. 24 qt + 23 (three groups of eight), one fp16
        // in the low half of each accumulator word; packed and staged so that every thread then
        // finds its own row's 16 policy columns and the expansion warp whole rows
        uint32_t acc[24];
#pragma unroll
        for (int jj = 0; jj < 3; ++jj)
            tmem_ld8(c.tm + TM_ACC + 24 * c.qt + 8 * jj, *reinterpret_cast<uint32_t(*)[8]>(&acc[8 * jj]));
        row_release_acc(c, 0);                           // waits for the loads
#pragma unroll
        for (int jj = 0; jj < 3; ++jj) {
            const int j = 3 * c.qt + jj;
            const uint32_t base = j < 8 ? stage_pol : stage_aux;
            sts128(base + sw_off(c.row, j & 7),
                   make_uint4(__byte_perm(acc[8 * jj], acc[8 * jj + 1], 0x5410),
                              __byte_perm(acc[8 * jj + 2], acc[8 * jj + 3], 0x5410),
                              __byte_perm(acc[8 * jj + 4], acc[8 * jj + 5], 0x5410),
                              __byte_perm(acc[8 * jj + 6], acc[8 * jj + 7], 0x5410)));
        }
    }
    board_sync(c);                                       // the board's 32 x 96 logits are staged
    {
        uint32_t lgw[8], aux[4] = {0u, 0u, 0u, 0u};
        {
            const uint4 v0 = lds128(stage_pol + sw_off(c.row, 2 * c.qt));
            const uint4 v1 = lds128(stage_pol + sw_off(c.row, 2 * c.qt + 1));
            lgw[0] = v0.x; lgw[1] = v0.y; lgw[2] = v0.z; lgw[3] = v0.w;
            lgw[4] = v1.x; lgw[5] = v1.y; lgw[6] = v1.z; lgw[7] = v1.w;
            if (c.qt == 0) {
                const uint4 va = lds128(stage_aux + sw_off(c.row, 0));        // columns 64..71
                aux[0] = va.x; aux[1] = va.y; aux[2] = va.z; aux[3] = va.w;
            }
        }
        uint32_t lg[8];
        const uint32_t bits = static_cast<uint32_t>(lw >> (16 * c.qt)) & 0xffffu;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            uint32_t v = lgw[i];
            if (!((bits >> (2 * i)) & 1u)) v = (v & 0xffff0000u) | 0xfc00u;
            if (!((bits >> (2 * i + 1)) & 1u)) v = (v & 0x0000ffffu) | 0xfc000000u;
            lg[i] = v;
        }
        if (c.valid && p.policy != nullptr) store_words<8>(p.policy + c.grow * 64 + 16 * c.qt, lg);
        if (p.prior != nullptr && c.qt == 1) {
            // the list is put together in this board's rows of the staging region's third block,
            // idle from the head product (which read it) to the next tile's first QKV staging
            expand_board(p, board, c.lane, c.valid, word, ctl, moves, stage_pol, stage_aux, c.row,
                         c.smem_gen + (c.sm_r - c.smem) + 32768u + 4096u * c.q);
        }
        if (c.qt == 0) {
            if (c.valid && p.promo != nullptr)
                *reinterpret_cast<uint2*>(p.promo + c.grow * 4) = make_uint2(aux[0], aux[1]);
            // value logits: the fp16 head outputs in columns 68, 69, 70
            float a = __low2float(as_h2(aux[2])), b = __high2float(as_h2(aux[2]));
            float d = __low2float(as_h2(aux[3]));
            if (p.vmode == 1) {
                // live tokens in slot order, one after the other (encoder.cu:1040-1057)
                float ta = 0.f, tb = 0.f, td = 0.f;
#pragma unroll 1
                for (int tt = 0; tt < kT; ++tt) {
                    const float at = __shfl_sync(0xffffffffu, a, tt), bt = __shfl_sync(0xffffffffu, b, tt);
                    const float dt = __shfl_sync(0xffffffffu, d, tt);
                    if ((alive >> tt) & 1u) { ta += at; tb += bt; td += dt; }
                }
                a = ta; b = tb; d = td;
                const int nlive = __popc(alive);
                const float inv = 1.0f / static_cast<float>(nlive > 0 ? nlive : 1);
                a *= inv; b *= inv; d *= inv;
            }
            if (p.vmode == 2) { a = pre[0]; b = pre[1]; d = pre[2]; }
            const bool writer = p.vmode != 0 ? c.lane == 0 : c.lane == (ctl < 0 ? 31 : 15);
            if (writer && c.valid && p.value != nullptr) {
                float v;
                if (p.n_value == 1) {
                    v = tanhf(a);
                } else {
                    const float m = fmaxf(a, fmaxf(b, d));
                    const float ea = expf(a - m), eb = expf(b - m), ec = expf(d - m);
                    v = (ec - ea) / (ea + eb + ec);
                }
                if (p.vmode != 0 && ctl < 0) v = -v;
                p.value[board] = v;
            }
        }
    }
    prof_mark<kDbg>(c, PH_HEAD);
}

template <bool kDbg, bool kRJ, int kAr>
__device__ __forceinline__ void row_warps_tile(RowCtx& c, const Params& p, int tile) {
    const int item = tile * 4 + c.q;
    c.valid = item < c.n;
    // with a leaf list the board is read from, and its outputs written to, its own place in the
    // staged arrays
    const int board = (c.valid && p.leaf_index != nullptr) ? __ldg(p.leaf_index + item) : item;
    c.grow = static_cast<long>(board) * kT + c.lane;
    const bool backbone = kDbg && p.x_in != nullptr;
    const uint32_t word = (c.valid && !backbone) ? p.boards[c.grow] : 0u;
    uint32_t alive = __ballot_sync(0xffffffffu, ((word >> 11) & 1u) == 0u);
    if (backbone && p.alive_in != nullptr)
        alive = __ballot_sync(0xffffffffu, c.valid ? p.alive_in[c.grow] != 0 : true);
    const int ctl = (c.valid && !backbone) ? static_cast<int>(p.control[board]) : 1;
    const int dbg = p.debug_stage;

    if (backbone) {
        // activations in (the reference's `encoder_forward`, encoder.cu:1752-1767): this token's
        // row of x becomes the residual stream as it is
        c.word = 0u; c.stm = 0; c.clk = 0; c.rp = 0;
#pragma unroll 1
        for (int u = 0; u < 2; ++u) {
            uint32_t e16[16];
            const uint4* src = reinterpret_cast<const uint4*>(p.x_in + c.grow * kD + 128 * u + 32 * c.qt);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint4 v = c.valid ? __ldg(src + k) : make_uint4(0u, 0u, 0u, 0u);
                e16[4 * k] = v.x; e16[4 * k + 1] = v.y; e16[4 * k + 2] = v.z; e16[4 * k + 3] = v.w;
            }
            tmem_st16(c.tm + TM_X + 64 * u + 16 * c.qt, e16);
        }
        tmem_wait_st();
    } else
    // ---- embedding: ((square + type_special) + color_turn) + (clock + rep), fp16
    //      (encoder.cu:817-889; nn/model.py:383-397), written to the residual stream ----
    {
        const int stm = ctl < 0;
        const int clk = min(max((ctl < 0 ? -ctl : ctl) - 1, 0), kNClock - 1);
        const int rp = min((c.valid && !backbone) ? static_cast<int>(p.rep[board]) : 0, kNRep - 1);
        c.word = word; c.stm = stm; c.clk = clk; c.rp = rp;
        const int sq = word & 63;
        const int ts = min(static_cast<int>(((word >> 6) & 7) * 2 + ((word >> 9) & 1)), kNTypeSpecial - 1);
        const int ct = ((word >> 10) & 1) * 2 + stm;
#pragma unroll 1
        for (int u = 0; u < 2; ++u) {
            const int col = 128 * u + 32 * c.qt;
            const uint4* e_sq = reinterpret_cast<const uint4*>(p.emb + (EMB_SQUARE + sq) * kD + col);
            const uint4* e_ts = reinterpret_cast<const uint4*>(p.emb + (EMB_TS + ts) * kD + col);
            const uint4* e_ct = reinterpret_cast<const uint4*>(p.emb + (EMB_CT + ct) * kD + col);
            const uint4* e_ck = reinterpret_cast<const uint4*>(p.emb + (EMB_CLOCK + clk) * kD + col);
            const uint4* e_rp = reinterpret_cast<const uint4*>(p.emb + (EMB_REP + rp) * kD + col);
            uint32_t e16[16];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint4 a = __ldg(e_sq + k), b = __ldg(e_ts + k), d = __ldg(e_ct + k);
                const uint4 e = __ldg(e_ck + k), f = __ldg(e_rp + k);
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
                const uint32_t dw[4] = {d.x, d.y, d.z, d.w}, ew[4] = {e.x, e.y, e.z, e.w};
                const uint32_t fw[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __half2 x = __hadd2(as_h2(aw[j]), as_h2(bw[j]));
                    x = __hadd2(x, as_h2(dw[j]));
                    x = __hadd2(x, __hadd2(as_h2(ew[j]), as_h2(fw[j])));
                    e16[4 * k + j] = as_u32(x);
                }
            }
            tmem_st16(c.tm + TM_X + 64 * u + 16 * c.qt, e16);
        }
        tmem_wait_st();
    }
    prof_mark<kDbg>(c, PH_EMBED);

    const int n_ph = 2 * p.n_layers;
#pragma unroll 1
    for (int ph = 0; ph <= n_ph; ++ph) {
        const int layer = ph >> 1;
        const bool odd = ph & 1;
        const bool dbgl = layer == p.debug_layer;
        const bool dump_x = (dbg == 9 && ph == 0) || (dbg == 2 && odd && dbgl) ||
                            (dbg == 10 && !odd && ph > 0 && layer - 1 == p.debug_layer);
        // This half-layer's scales and biases (the final norm's affine and value rows at the end)
        // are asked into L1 now, a norm ahead of their first use: the eight layers' 37 KB do not
        // stay there from one tile to the next beside 228 KB of shared memory.
        {
            const int t = 32 * (c.q + 4 * c.qt) + c.lane;
            if (ph == n_ph) {
                if (t < static_cast<int>(kTailBytes / 128)) prefetch_l1(reinterpret_cast<const uint8_t*>(p.tail) + 128 * t);
            } else if (t < kLparamStride / 128) {
                prefetch_l1(p.lparams + static_cast<size_t>(layer) * kLparamStride + 128 * t);
            }
        }
        if (ph == n_ph) {
            ln_stage<kDbg, kRJ, kAr>(c, p, true, dump_x, dbg == 8, false, -1);
            row_publish(c, B_A_READY);                   // the head product's A operand
            break;
        }
        const bool cap = layer == p.cap_layer;
        // re-injection site of this norm: every norm when both inject, attention norms only else
        const int site = !kRJ ? -1 : (p.rj_mode == 2 ? ph : (odd ? -1 : layer));
        const float sa = ln_stage<kDbg, kRJ, kAr>(c, p, false, dump_x, dbgl && dbg == (odd ? 3 : 1),
                                                cap && p.cap_op == (odd ? BF_OP_FF1 : BF_OP_QKV), site,
                                                kAr == kArF16 || ((kAr == kArE4M3 || kAr == kArI8Ffn) && !odd));
        row_publish(c, B_A_READY);

        const uint8_t* lpb = p.lparams + static_cast<size_t>(layer) * kLparamStride;
        LayerParams lp;
        lp.sw_qkv = reinterpret_cast<const float*>(lpb + LP_SW_QKV);
        lp.sw_o = reinterpret_cast<const float*>(lpb + LP_SW_O);
        lp.sw_ff1 = reinterpret_cast<const float*>(lpb + LP_SW_FF1);
        lp.sw_ff2 = reinterpret_cast<const float*>(lpb + LP_SW_FF2);
        lp.b_qkv = reinterpret_cast<const __half*>(lpb + LP_B_QKV);
        lp.b_o = reinterpret_cast<const __half*>(lpb + LP_B_O);
        lp.b_ff1 = reinterpret_cast<const __half*>(lpb + LP_B_FF1);
        lp.b_ff2 = reinterpret_cast<const __half*>(lpb + LP_B_FF2);
        if (!odd) attention_block<kDbg, kAr>(c, p, lp, sa, c.valid ? alive : 0xffffffffu, cap, dbgl);
        else if constexpr (kAr == kArF16) ffn_block_f16<kDbg>(c, p, lp);
        else      ffn_block<kDbg, kAr>(c, p, lp, sa, cap);
    }

    head_epilogue<kDbg>(c, p, board, word, ctl, alive);
}

}  // namespace bf
#include "bf_encoder_one.cuh"
namespace bf {

// ------------------------------------------------------------------------------------------
// Producer: streams the packed weight stage images through the ring.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t uses(uint32_t cnt, uint32_t slots, uint32_t s) {
    return (cnt + slots - 1 - s) / slots;
}

template <int kAr>
__device__ __forceinline__ void producer_loop(uint32_t smem, volatile int* abort_flag, const Params& p,
                                           int first_tile, int tile_step, int n_tiles) {
    using C = Cfg<kAr>;
    constexpr uint32_t kQS = C::kQSlots, kRS = C::kRSlots;
    uint32_t qi = 0, ri = 0;   // stages issued into the QKV ring / the 16 KB ring
    for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
        const uint8_t* src = p.wstream;
        for (int layer = 0; layer < p.n_layers; ++layer) {
            {
                // the two rings share memory: the 16 KB ring must be drained first
                for (uint32_t s = 0; s < kRS; ++s)
                    mbar_wait(bar_addr(smem, B_WR_EMPTY + s), (uses(ri, kRS, s) - 1u) & 1u, abort_flag, kErrProducer);
                for (int st = 0; st < 4 * C::kQkvSlabs; ++st, ++qi) {
                    const uint32_t s = qi % kQS;
                    mbar_wait(bar_addr(smem, B_WQ_EMPTY + s), (qi / kQS - 1u) & 1u, abort_flag, kErrProducer);
                    mbar_arrive_expect_tx(bar_addr(smem, B_WQ_FULL + s), kQStage);
                    bulk_g2s(smem + C::SM_RING + s * kQStage, src, kQStage, bar_addr(smem, B_WQ_FULL + s));
                    src += kQStage;
                }
                for (uint32_t s = 0; s < kQS; ++s)
                    mbar_wait(bar_addr(smem, B_WQ_EMPTY + s), (uses(qi, kQS, s) - 1u) & 1u, abort_flag, kErrProducer);
            }
            // out-projection (2 units) and the 16 FFN units
            const int n_st = 2 * C::kOutSlabs + 16 * C::kFfnSlabs;
            const uint32_t bytes = kRStage;
            for (int st = 0; st < n_st; ++st, ++ri) {
                const uint32_t s = ri % kRS;
                mbar_wait(bar_addr(smem, B_WR_EMPTY + s), (ri / kRS - 1u) & 1u, abort_flag, kErrProducer);
                mbar_arrive_expect_tx(bar_addr(smem, B_WR_FULL + s), bytes);
                bulk_g2s(smem + C::SM_RING + s * kRStage, src, bytes, bar_addr(smem, B_WR_FULL + s));
                src += bytes;
            }
        }
        // the head matrix: four K-slabs of 96 rows in 16 KB slots
        for (uint32_t st = 0; st < kHeadStages; ++st, ++ri) {
            const uint32_t s = ri % kRS;
            mbar_wait(bar_addr(smem, B_WR_EMPTY + s), (ri / kRS - 1u) & 1u, abort_flag, kErrProducer);
            mbar_arrive_expect_tx(bar_addr(smem, B_WR_FULL + s), kHeadStage);
            bulk_g2s(smem + C::SM_RING + s * kRStage, src, kHeadStage, bar_addr(smem, B_WR_FULL + s));
            src += kHeadStage;
        }
    }
    // Every copy issued has been waited for by the MMA issuer on the normal path.  After a
    // time-out some may still be in flight: give them a bounded while to land before the
    // CTA's shared memory goes away.
    if (*abort_flag != 0) {
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) { }
    }
}

// ------------------------------------------------------------------------------------------
// MMA issuer: one thread walks the static GEMM schedule.
// ------------------------------------------------------------------------------------------
struct MmaState {
    uint32_t qc, rc;          // weight stages consumed from each ring
    uint32_t accn[2];         // units issued into each accumulator slot
    uint32_t aready, a2n[2];  // operand-ready phases consumed
};
enum { kKindI8 = 0, kKindF16 = 1, kKindF8 = 2 };

// One GEMM unit: `n_stages` K-slabs of 128 bytes, 4 MMAs each.
template <int kAr>
__device__ __forceinline__ void mma_unit(uint32_t smem, volatile int* abort_flag, MmaState& st,
                                         uint32_t tmem_d, int slot, uint32_t a_base, bool qring,
                                         int n_stages, uint32_t idesc, int kind, bool pre = false) {
    using C = Cfg<kAr>;
    // `pre`: mma_prewait has already seen the slot free and the first weight stage in place
    // (the fences that order the MMAs after what those waits saw: after a pre-wait it is the
    // operand wait's own fence, which comes later than both)
    if (!pre) {
        mbar_wait(bar_addr(smem, B_ACC_EMPTY + slot), (st.accn[slot] - 1u) & 1u, abort_flag, kErrMmaAcc);
        tc_fence_after();
    }
    for (int s = 0; s < n_stages; ++s) {
        uint32_t w_empty, w_addr;
        const bool seen = pre && s == 0;
        if (qring) {
            const uint32_t k = st.qc % C::kQSlots;
            if (!seen) mbar_wait(bar_addr(smem, B_WQ_FULL + k), (st.qc / C::kQSlots) & 1u, abort_flag, kErrMmaWeights);
            w_empty = bar_addr(smem, B_WQ_EMPTY + k); w_addr = smem + C::SM_RING + k * kQStage;
            st.qc++;
        } else {
            const uint32_t k = st.rc % C::kRSlots;
            if (!seen) mbar_wait(bar_addr(smem, B_WR_FULL + k), (st.rc / C::kRSlots) & 1u, abort_flag, kErrMmaWeights);
            w_empty = bar_addr(smem, B_WR_EMPTY + k); w_addr = smem + C::SM_RING + k * kRStage;
            st.rc++;
        }
        if (!seen) tc_fence_after();
        const uint64_t ad = umma_desc_k128(a_base + s * 16384), bd = umma_desc_k128(w_addr);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t accumulate = (s > 0 || k > 0) ? 1u : 0u;
            if (kind == kKindF16)     umma_f16(tmem_d, ad + 2 * k, bd + 2 * k, idesc, accumulate);
            else if (kind == kKindF8) umma_f8(tmem_d, ad + 2 * k, bd + 2 * k, idesc, accumulate);
            else                      umma_i8(tmem_d, ad + 2 * k, bd + 2 * k, idesc, accumulate);
        }
        tc_commit(w_empty);
    }
    tc_commit(bar_addr(smem, B_ACC_FULL + slot));
    st.accn[slot]++;
}

// What a unit needs besides its A operand -- its accumulator slot handed back, its first weight
// stage in place -- waited for BEFORE the issuer blocks on the operand barrier: both come from
// work that is long done by then, and a wait costs a shared-memory round trip even when it
// succeeds at once, which would otherwise sit between the operand's arrival and the first MMA.
template <int kAr>
__device__ __forceinline__ void mma_prewait(uint32_t smem, volatile int* abort_flag, const MmaState& st,
                                            int slot, bool qring) {
    using C = Cfg<kAr>;
    mbar_wait(bar_addr(smem, B_ACC_EMPTY + slot), (st.accn[slot] - 1u) & 1u, abort_flag, kErrMmaAcc);
    if (qring) {
        const uint32_t k = st.qc % C::kQSlots;
        mbar_wait(bar_addr(smem, B_WQ_FULL + k), (st.qc / C::kQSlots) & 1u, abort_flag, kErrMmaWeights);
    } else {
        const uint32_t k = st.rc % C::kRSlots;
        mbar_wait(bar_addr(smem, B_WR_FULL + k), (st.rc / C::kRSlots) & 1u, abort_flag, kErrMmaWeights);
    }
}

__device__ __forceinline__ void mma_wait_operand(uint32_t smem, volatile int* abort_flag, int bar_idx,
                                                 uint32_t& cnt) {
    mbar_wait(bar_addr(smem, bar_idx), cnt & 1u, abort_flag, kErrMmaOperand);
    cnt++;
    tc_fence_after();
}

// Step over `n_stages` weight stages that the other issuer consumes: wait for each one's arrival
// and release it as a consumer would.  A slot is refilled when both issuers have released it, so
// both see every filling of every slot in order and neither can fall a phase behind on the ring's
// barriers or run a phase ahead (a parity wait tells only the current phase from the one before,
// and two bulk copies need not complete in the order they were issued).
template <int kAr>
__device__ __forceinline__ void mma_pass_over(uint32_t smem, volatile int* abort_flag, MmaState& st, int n_stages) {
    using C = Cfg<kAr>;
#pragma unroll 1
    for (int i = 0; i < n_stages; ++i) {
        const uint32_t k = st.rc % C::kRSlots;
        mbar_wait(bar_addr(smem, B_WR_FULL + k), (st.rc / C::kRSlots) & 1u, abort_flag, kErrMmaWeights);
        mbar_arrive(bar_addr(smem, B_WR_EMPTY + k));
        st.rc++;
    }
}

// Two threads (lane 0 of two warps) share the schedule: issuing one unit costs a thread well
// over twice the unit's time on the tensor pipe (barrier waits, descriptors, a full MMA queue),
// and the units of a step come in pairs -- the two 128-wide halves of an out-projection, of a
// hidden chunk, of an ff2 chunk -- that are independent of one another.  Issuer `who` takes the
// half-`who` unit of every pair (its accumulator slot is slot `who`) and steps over the other
// half's weight stages; the QKV units, which follow one another on one accumulator, and the head
// product are issuer 0's.  Both issuers wait for every phase of the operand barriers in order,
// needed or not, because a parity wait must not fall a phase behind; for the same reason the
// other half's weight stages are passed over one by one (mma_pass_over).  In the fp16 arithmetic's
// FFN (ff1 units on slot 0, one running pair of ff2 accumulators) issuer 0 takes the ff1 units
// and issuer 1 the ff2 units; only issuer 1 waits on the hidden-chunk barrier there.
template <int kAr>
__device__ __forceinline__ void mma_loop(uint32_t smem, uint32_t tmem, volatile int* abort_flag,
                                      const Params& p, int first_tile, int tile_step, int n_tiles, int who) {
    using C = Cfg<kAr>;
    MmaState st = {0, 0, {0, 0}, 0, {0, 0}};
    // int8: every weight GEMM is s8/u8 x s8.  e4m3: QKV and out-projection are fp16 x fp16 with
    // fp16 accumulators (the bits of the reference's mma.sync), the FFN is e4m3 x e4m3 with fp32
    // accumulators (the reference's fp16-accumulate e4m3 mma.sync has no bit-equal on tcgen05).
    constexpr bool kHalfA = kAr != kArInt8;
    constexpr uint32_t kI_H128 = umma_idesc(kAccF16, kFmtF16, kFmtF16, 128, 128);
    constexpr uint32_t kI_QKV = C::kQkvF16 ? umma_idesc(kAccF16, kFmtF16, kFmtF16, 128, 192)
                                       : umma_idesc(kAccS32, kFmtS8, kFmtS8, 128, 192);
    constexpr uint32_t kI_OUT = C::kOutF16 ? kI_H128 : umma_idesc(kAccS32, kFmtS8, kFmtS8, 128, 128);
    constexpr uint32_t kI_FF1 = kAr == kArE4M3 ? umma_idesc(kAccF32, kFmtE4M3, kFmtE4M3, 128, 128)
                              : kAr == kArF16 ? kI_H128 : umma_idesc(kAccS32, kFmtS8, kFmtS8, 128, 128);
    constexpr uint32_t kI_FF2 = kAr == kArE4M3 ? umma_idesc(kAccF32, kFmtE4M3, kFmtE4M3, 128, 128)
                              : kAr == kArF16 ? kI_H128 : umma_idesc(kAccS32, kFmtU8, kFmtS8, 128, 128);
    constexpr int kQkvKind = C::kQkvF16 ? kKindF16 : kKindI8, kOutKind = C::kOutF16 ? kKindF16 : kKindI8;
    constexpr int kFfnKind = kAr == kArE4M3 ? kKindF8 : (kAr == kArF16 ? kKindF16 : kKindI8);
    const uint32_t acc0 = tmem + TM_ACC, acc1 = tmem + TM_ACC + 128;
    const uint32_t sm_a = smem + C::SM_A, sm_r = smem + C::SM_R;
    (void)kHalfA;
    for (int tile = first_tile; tile < n_tiles; tile += tile_step) {
        for (int layer = 0; layer < p.n_layers; ++layer) {
            if (who == 0) mma_prewait<kAr>(smem, abort_flag, st, 0, true);
            mma_wait_operand(smem, abort_flag, B_A_READY, st.aready);          // LN1 output
            if (who == 0)
                for (int j = 0; j < 4; ++j)
                    mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_a, true, C::kQkvSlabs, kI_QKV, kQkvKind, j == 0);
            if (who == 1) mma_pass_over<kAr>(smem, abort_flag, st, C::kOutSlabs);
            mma_prewait<kAr>(smem, abort_flag, st, who, false);
            mma_wait_operand(smem, abort_flag, B_A_READY, st.aready);          // attention output
            if (who == 0) {
                mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_a, false, C::kOutSlabs, kI_OUT, kOutKind, true);
                mma_pass_over<kAr>(smem, abort_flag, st, C::kOutSlabs);
            } else {
                mma_unit<kAr>(smem, abort_flag, st, acc1, 1, sm_a, false, C::kOutSlabs, kI_OUT, kOutKind, true);
            }
            // the FFN's first unit of this issuer (every arithmetic: ff1, chunk 0, half `who`)
            bool ffn_pre = false;
            if constexpr (kAr != kArF16) {
                if (who == 1) mma_pass_over<kAr>(smem, abort_flag, st, 2);
                mma_prewait<kAr>(smem, abort_flag, st, who, false);
                ffn_pre = true;
            }
            mma_wait_operand(smem, abort_flag, B_A_READY, st.aready);          // LN2 output
            if constexpr (kAr == kArF16) {
                // fp16 FFN: ff1 units go into slot 0; once the rows have written a hidden chunk,
                // its two ff2 units follow, whose accumulators (the idle
                // attention-output columns for half 0, slot 1 for half 1) run on through all
                // four chunks; one commit per chunk on accumulator barrier 1 tells the rows
                // that the hidden buffer is free again, the last one that the sums are done
                // issue order (= the packed weight order): F1 c0 j0, F1 c0 j1, then per chunk c:
                // F1 c+1 j0 (so that it runs under the rows' epilogue of F1 c j1), F2 c j0, F2 c j1,
                // F1 c+1 j1
                // issuer 0 takes the ff1 units (slot 0), issuer 1 the ff2 units; each steps over
                // the other's weight stages
                auto pass_over = [&](int n_stages) { mma_pass_over<kAr>(smem, abort_flag, st, n_stages); };
                if (who == 0) {
                    mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_a, false, 4, kI_FF1, kKindF16);
                    mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_a, false, 4, kI_FF1, kKindF16);
#pragma unroll 1
                    for (int ch = 0; ch < 4; ++ch) {
                        if (ch < 3) mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_a, false, 4, kI_FF1, kKindF16);
                        pass_over(8);
                        if (ch < 3) mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_a, false, 4, kI_FF1, kKindF16);
                    }
                } else {
                pass_over(8);
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    if (ch < 3) pass_over(4);
                    mma_wait_operand(smem, abort_flag, B_A2_READY, st.a2n[0]);
                    if (ch == 0) {
                        mbar_wait(bar_addr(smem, B_ACC_EMPTY + 1), (st.accn[1] - 1u) & 1u, abort_flag, kErrMmaAcc);
                        tc_fence_after();
                    }
#pragma unroll 1
                    for (int jh = 0; jh < 2; ++jh) {
                        const uint32_t dst = jh ? acc1 : tmem + TM_OY;
#pragma unroll 1
                        for (int sl = 0; sl < 4; ++sl) {
                            const uint32_t k = st.rc % C::kRSlots;
                            mbar_wait(bar_addr(smem, B_WR_FULL + k), (st.rc / C::kRSlots) & 1u, abort_flag, kErrMmaWeights);
                            st.rc++;
                            tc_fence_after();
                            const uint64_t ad = umma_desc_k128(sm_r + sl * 16384);
                            const uint64_t bd = umma_desc_k128(smem + C::SM_RING + k * kRStage);
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk)
                                umma_f16(dst, ad + 2 * kk, bd + 2 * kk, kI_FF2, (ch > 0 || sl > 0 || kk > 0) ? 1u : 0u);
                            tc_commit(bar_addr(smem, B_WR_EMPTY + k));
                        }
                    }
                    tc_commit(bar_addr(smem, B_ACC_FULL + 1));
                    if (ch < 3) pass_over(4);
                }
                st.accn[1]++;
                }
            } else {
            // FFN units in the order the weight stream was packed (pack.py: FFN_UNITS)
#pragma unroll 1
            for (int u = 0; u < 16; ++u) {
                // kind/chunk of unit u: pairs (u>>1): F1 0, F1 1, F2 0, F1 2, F2 1, F1 3, F2 2, F2 3
                const int pr = u >> 1, jh = u & 1;
                if (jh != who) {                                          // the other issuer's unit
                    if (!(u == 0 && ffn_pre)) mma_pass_over<kAr>(smem, abort_flag, st, 2);   // (unit 0: passed above)
                    continue;
                }
                const int kind2 = (0xD4 >> pr) & 1;                       // 0b11010100
                const int ch = kind2 ? ((0x32010000u >> (4 * pr)) & 0xF) : ((0x00302010u >> (4 * pr)) & 0xF);
                if (kind2) {
                    mma_prewait<kAr>(smem, abort_flag, st, jh, false);
                    mma_wait_operand(smem, abort_flag, B_A2_READY + (ch & 1), st.a2n[ch & 1]);
                    mma_unit<kAr>(smem, abort_flag, st, jh ? acc1 : acc0, jh, sm_r + (ch & 1) * 32768,
                                   false, 2, kI_FF2, kFfnKind, true);
                } else {
                    mma_unit<kAr>(smem, abort_flag, st, jh ? acc1 : acc0, jh, sm_a, false, 2, kI_FF1, kFfnKind,
                                   pr == 0 && ffn_pre);
                }
            }
            }
        }
        // heads: [128 x 256] x [96 x 256]^T in fp16 with fp16 accumulators, sixteen steps of
        // sixteen in rising order -- the bits of the reference's fp16-accumulate mma.sync head
        // product (encoder.cu:309-352, 918-927); A is the final norm's output in the staging region
        if (who == 0) mma_prewait<kAr>(smem, abort_flag, st, 0, false);
        mma_wait_operand(smem, abort_flag, B_A_READY, st.aready);
        if (who == 0)
            mma_unit<kAr>(smem, abort_flag, st, acc0, 0, sm_r, false, kHeadStages,
                          umma_idesc(kAccF16, kFmtF16, kFmtF16, 128, 96), kKindF16, true);
        else
            mma_pass_over<kAr>(smem, abort_flag, st, kHeadStages);
    }
}

// ------------------------------------------------------------------------------------------
// `kForm`: 0 = four boards per tile; 1 = the small-batch form, one board per tile with its rows
// replicated in the four lane quadrants (bf_encoder_one.cuh; plain int8 evaluation only); 2 = chosen
// when the kernel starts, by the number of positions it finds (a leaf list's length is only known
// on the device): one board per tile if every board gets a CTA of its own, else four.
enum { kFormFour = 0, kFormOne = 1, kFormByCount = 2 };
template <bool kDbg, bool kRJ, int kAr, int kForm = kFormFour>
__global__ void __launch_bounds__(kThreads, 1) encoder_kernel(const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem = smem_u32(sm);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + SM_MISC + 4);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + SM_MISC);

    if (threadIdx.x == 0) {
        for (int i = 0; i < B_COUNT; ++i) {
            const bool many = (i >= B_ACC_EMPTY && i < B_ACC_EMPTY + 2) || i >= B_A_READY;
            // a slot of the 16 KB weight ring is released by both MMA issuers
            const bool both = i >= B_WR_EMPTY && i < B_WR_EMPTY + 7;
            mbar_init(bar_addr(smem, i), many ? kRowWarps : (both ? 2 : 1));
        }
        *abort_flag = 0;
        for (int i = 0; i < 16; ++i) reinterpret_cast<long long*>(sm + SM_PROF)[i] = 0;
        fence_barrier_init();
    }
    if (warp == kMmaWarp) {
        tmem_alloc(smem + SM_MISC, TM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    // the number of positions: the launch's own, or what the device-side leaf count says now
    // (clamped to the capacity the grid was sized for); every role reads the same word
    int n_eval = p.n;
    if (p.leaf_count != nullptr) n_eval = min(max(__ldg(p.leaf_count), 0), p.n);
    const bool one = kForm == kFormOne || (kForm == kFormByCount && n_eval <= static_cast<int>(gridDim.x));
    const int n_tiles = one ? n_eval : (n_eval + 3) / 4;
    if (warp < kRowWarps) {
        RowCtx c;
        c.n = n_eval;
        c.lane = lane; c.q = warp & 3; c.qt = warp >> 2; c.row = 32 * c.q + lane;
        c.smem = smem; c.smem_gen = sm;
        c.sm_a = smem + Cfg<kAr>::SM_A; c.sm_r = smem + Cfg<kAr>::SM_R;
        c.tm = tmem + (static_cast<uint32_t>(32 * c.q) << 16);
        c.abort_flag = abort_flag; c.xpar = 0; c.full0 = c.full1 = 0;
        c.one2 = pk2(p.one, p.one);
        c.prof_on = kDbg && p.prof != nullptr && threadIdx.x == 0;
        c.t_last = c.prof_on ? clock64() : 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
            if constexpr (kForm == kFormFour) {
                row_warps_tile<kDbg, kRJ, kAr>(c, p, tile);
            } else {
                if (one)
                    one::row_warps_tile(c, p, tile, [&](RowCtx& cc, int board, uint32_t word, int ctl, uint32_t alive) {
                        head_epilogue<false>(cc, p, board, word, ctl, alive);
                    });
                else
                    row_warps_tile<kDbg, kRJ, kAr>(c, p, tile);
            }
        }
    } else if (warp == kProducerWarp) {
        if (lane == 0) producer_loop<kAr>(smem, abort_flag, p, blockIdx.x, gridDim.x, n_tiles);
    } else {
        if (lane == 0) mma_loop<kAr>(smem, tmem, abort_flag, p, blockIdx.x, gridDim.x, n_tiles, warp - kMmaWarp);
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == kMmaWarp) tmem_dealloc(tmem, TM_COLS);
    if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(p.status, 0, *abort_flag);
    if (kDbg && threadIdx.x == 0 && p.prof != nullptr)
        for (int i = 0; i < PH_COUNT; ++i)
            atomicAdd(p.prof + i, static_cast<unsigned long long>(reinterpret_cast<long long*>(sm + SM_PROF)[i]));
}

// ------------------------------------------------------------------------------------------
// CUDA-core probe: what one SM sustains on the element-wise building blocks of the row warps when
// nothing else is in the way -- operands in shared memory, sixteen warps resident as in the
// evaluator, no tensor-memory loads, no exchanges, no barriers.  The same device functions the
// evaluator calls.  Block 0: ff1 epilogue (s32 -> descale -> bias + ReLU -> row maximum -> u8);
// 1: descale + bias -> fp16 (QKV and out-projection epilogues); 2: ff2 step (descale, fused add
// to the fp16 running total); 3: norm statistics (sum, sum of squares, minimum, maximum); 4:
// normalise -> fp16 -> s8; 5: fp16 -> int8 quantisation alone; 8-11: the cheaper forms of blocks 0,
// 4, 1 and 2 that a not-bit-exact arithmetic could use (one combined scale, the requantisation in
// fp16 or fused into the normalise), to measure what giving up the reference's bits would buy.
// 32 elements per thread and pass.
// The host entry also runs block 0 with eight and with thirty-two warps resident (its blocks 6
// and 7), which shows how much a different number of row warps could change.
// ------------------------------------------------------------------------------------------
template <int kBlock, int kProbeThreads>
__global__ void __launch_bounds__(kProbeThreads, 1) elementwise_probe_kernel(const __half* bias, float sa, float sw,
                                                                              float one, int iters, float* out) {
    extern __shared__ uint32_t probe_sm[];
    const int tid = threadIdx.x;
    for (int i = tid; i < 32 * kProbeThreads; i += kProbeThreads) probe_sm[i] = 0x3c003800u + ((i * 2654435761u) >> 20);
    __syncthreads();
    const uint64_t one2 = pk2(one, one), sa2 = pk2(sa, sa), sw2 = pk2(sw, sw);
    float m = 0.f;
    uint32_t keep = 0;
    uint64_t sum2 = pk2(0.f, 0.f), sq2 = pk2(0.f, 0.f);
    __half2 mn = __float2half2_rn(65504.0f), mx = __float2half2_rn(-65504.0f);
    uint32_t run[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) run[i] = 0;
    for (int it = 0; it < iters; ++it) {
        uint32_t acc[32], o[16];
        if (kBlock <= 2 || kBlock == 8 || kBlock >= 10) {
#pragma unroll
            for (int k = 0; k < 32; ++k) acc[k] = probe_sm[k * kProbeThreads + tid] + it;
        } else {
#pragma unroll
            for (int k = 0; k < 16; ++k) o[k] = probe_sm[k * kProbeThreads + tid] ^ (it & 1);
        }
        if (kBlock == 0) {
            descale<32, true, kAccInt>(acc, sa, sw, bias, o);
            const float am = amax_h2<16>(o, false);
            m = fmaxf(m, am);
            const float inv = 255.0f / fmaxf(am, 1e-3f);
            const uint4 a = quant16(&o[0], inv, one2), b = quant16(&o[8], inv, one2);
            keep ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w;
        } else if (kBlock == 1) {
            descale<32, false, kAccInt>(acc, sa, sw, bias, o);
#pragma unroll
            for (int k = 0; k < 16; ++k) probe_sm[(16 + k) * kProbeThreads + tid] = o[k];
        } else if (kBlock == 2) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                uint64_t f = pk2(static_cast<float>(static_cast<int>(acc[2 * i])),
                                 static_cast<float>(static_cast<int>(acc[2 * i + 1])));
                f = fma2(mul2(f, sa2), sw2, h2_to_f2(run[i]));
                run[i] = f2_to_h2(f);
            }
        } else if (kBlock == 3) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint64_t f = h2_to_f2(o[i]);
                sum2 = add2(sum2, f);
                sq2 = fma2(f, f, sq2);
                mn = __hmin2(mn, as_h2(o[i]));
                mx = __hmax2(mx, as_h2(o[i]));
            }
        } else if (kBlock == 4) {
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = f2_to_h2(mul2(add2(h2_to_f2(o[i]), sa2), sw2));
            const uint4 a = quant16(&o[0], sa, one2), b = quant16(&o[8], sa, one2);
            keep ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w;
        } else if (kBlock == 5) {
            const uint4 a = quant16(&o[0], sa, one2), b = quant16(&o[8], sa, one2);
            keep ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w;
        } else if (kBlock == 8) {
            // ff1 epilogue, cheaper form: one combined scale, bias + ReLU as now, the u8
            // requantisation in fp16 (the rounding add on 1024 leaves the integer in the low
            // mantissa bits of each half: one packed fma and a quarter of a byte permute per
            // element instead of two conversions, a multiply, an fma and three quarters)
            const uint4* b4 = reinterpret_cast<const uint4*>(bias);
            const float s = sa * sw;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 bv = __ldg(b4 + v);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = 4 * v + k;
                    const uint64_t f = pk2(__fmul_rn(static_cast<float>(static_cast<int>(acc[2 * i])), s),
                                           __fmul_rn(static_cast<float>(static_cast<int>(acc[2 * i + 1])), s));
                    o[i] = hfma2_relu(f2_to_h2(f), 0x3C003C00u, bw[k]);
                }
            }
            const float am = amax_h2<16>(o, false);
            m = fmaxf(m, am);
            const __half2 inv = __float2half2_rn(255.0f / fmaxf(am, 1e-3f)), magic = __float2half2_rn(1024.0f);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                uint32_t q[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) q[j] = as_u32(__hfma2(as_h2(o[4 * k + j]), inv, magic));
                keep ^= __byte_perm(q[0], q[1], 0x6420) ^ __byte_perm(q[2], q[3], 0x6420);
            }
        } else if (kBlock == 9) {
            // normalise + s8 quantise, cheaper form: (x - mean) * rstd * inv and the rounding add as
            // one packed fma on the converted input
            const uint64_t a2 = pk2(sw, sw), b2 = pk2(12582912.0f + sa, 12582912.0f + sa);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float a0, a1, b0, b1, c0, c1, d0, d1;
                upk2(fma2(h2_to_f2(o[4 * k]), a2, b2), a0, a1);
                upk2(fma2(h2_to_f2(o[4 * k + 1]), a2, b2), b0, b1);
                upk2(fma2(h2_to_f2(o[4 * k + 2]), a2, b2), c0, c1);
                upk2(fma2(h2_to_f2(o[4 * k + 3]), a2, b2), d0, d1);
                keep ^= pack4(__float_as_uint(a0), __float_as_uint(a1), __float_as_uint(b0), __float_as_uint(b1)) ^
                        pack4(__float_as_uint(c0), __float_as_uint(c1), __float_as_uint(d0), __float_as_uint(d1));
            }
        } else if (kBlock == 10) {
            // descale + bias to fp16, cheaper form: one combined scale
            const uint4* b4 = reinterpret_cast<const uint4*>(bias);
            const float s = sa * sw;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const uint4 bv = __ldg(b4 + v);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = 4 * v + k;
                    const uint64_t f = pk2(__fmul_rn(static_cast<float>(static_cast<int>(acc[2 * i])), s),
                                           __fmul_rn(static_cast<float>(static_cast<int>(acc[2 * i + 1])), s));
                    probe_sm[(16 + i) * kProbeThreads + tid] = as_u32(__hadd2(as_h2(f2_to_h2(f)), as_h2(bw[k])));
                }
            }
        } else {
            // ff2 step, cheaper form: one combined scale in the fused add to the running total
            const float s = sa * sw;
            const uint64_t s2 = pk2(s, s);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const uint64_t f = pk2(static_cast<float>(static_cast<int>(acc[2 * i])),
                                       static_cast<float>(static_cast<int>(acc[2 * i + 1])));
                run[i] = f2_to_h2(fma2(f, s2, h2_to_f2(run[i])));
            }
        }
    }
    float a, b, c, d;
    upk2(sum2, a, b);
    upk2(sq2, c, d);
#pragma unroll
    for (int i = 0; i < 16; ++i) keep ^= run[i];
    out[blockIdx.x * kProbeThreads + tid] =
        m + a + b + c + d + __low2float(mn) + __high2float(mx) + __uint_as_float(keep & 0xffu);
}

// ------------------------------------------------------------------------------------------
// Tensor-pipe probe: what `tcgen05.mma kind::i8` sustains when nothing else is in the way.
// One CTA per SM; operands (pseudo-random bytes) sit in shared memory, accumulators in tensor
// memory; one thread issues `iters` groups of four M=128, N=256, K=32 MMAs back to back into two
// alternating accumulators, commits once and waits (bounded).  The counterpart of the
// reference's register-resident mma loop (csrc/fp8_loop.cu), used as the measured int8
// denominator of the roofline.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1) i8_peak_kernel(int iters, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem = smem_u32(sm);
    // layout: A [128 rows][128 B] at 0, B [256 rows][128 B] at 16384, barrier at 49152
    constexpr uint32_t kB = 16384, kBar = 49152;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kBar + 68);
    if (threadIdx.x == 0) {
        mbar_init(smem + kBar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if ((threadIdx.x >> 5) == 0) { tmem_alloc(smem + kBar + 68, 512); tmem_relinquish(); }
    uint32_t h = 0x9E3779B9u * (threadIdx.x + 1u) + blockIdx.x;
    for (uint32_t i = threadIdx.x; i < (kB + 32768u) / 4u; i += blockDim.x) {
        h = h * 1664525u + 1013904223u;
        reinterpret_cast<uint32_t*>(sm)[i] = h ^ (h >> 13);
    }
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = umma_idesc(kAccS32, kFmtS8, kFmtS8, 128, 256);
        const uint64_t ad = umma_desc_k128(smem), bd = umma_desc_k128(smem + kB);
        for (int it = 0; it < iters; ++it) {
            const uint32_t d = tmem + ((it & 1) ? 256u : 0u);
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_i8(d, ad + 2 * k, bd + 2 * k, idesc, (it > 1 || k > 0) ? 1u : 0u);
        }
        tc_commit(smem + kBar);
        mbar_wait(smem + kBar, 0, abort_flag, kErrMmaAcc);
        tc_fence_after();
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if ((threadIdx.x >> 5) == 0) tmem_dealloc(tmem, 512);
    if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

// ------------------------------------------------------------------------------------------
// Time-out self test: one thread waits on an mbarrier that nothing ever arrives on, through the
// same bounded wait every role of the evaluator uses.  The wait gives up after its cycle limit,
// the abort flag carries the code, the kernel returns normally and the host reads the status:
// the path a lost arrival takes in the real kernel, exercised without faulting anything.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(64, 1) timeout_kernel(int code, int* status, long long* waited) {
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    const uint32_t b = smem_u32(&bar);
    if (threadIdx.x == 0) {
        mbar_init(b, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const long long t0 = clock64();
        const bool ok = mbar_wait(b, 0, &abort_flag, code);
        *waited = clock64() - t0;
        if (ok) atomicCAS(status, 0, -1);          // cannot happen: nothing arrives
    }
    // a second waiter sees the flag and returns at once instead of waiting its own limit out
    __syncthreads();
    if (threadIdx.x == 32) {
        const long long t0 = clock64();
        mbar_wait(b, 0, &abort_flag, code + 100);
        waited[1] = clock64() - t0;
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag != 0) atomicCAS(status, 0, abort_flag);
}

// ------------------------------------------------------------------------------------------
// Tensor-core self test: one tile, one GEMM, no network.
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128, 1) selftest_kernel(int mode, const uint8_t* a, const uint8_t* w,
                                                          uint32_t* out, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem = smem_u32(sm);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, row = threadIdx.x;
    const int n = mode == 2 ? 192 : (mode == 3 ? 96 : 128);
    const int slabs = mode == 3 ? 4 : 2;
    const uint32_t w_stage = n * 128;
    // layout: A slabs at 0 (slabs x 16 KB), W at 65536, barriers at 163840
    constexpr uint32_t kW = 65536, kBar = 163840;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + kBar + 64);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + kBar + 68);
    if (threadIdx.x == 0) {
        mbar_init(smem + kBar, 1);
        mbar_init(smem + kBar + 8, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 0) { tmem_alloc(smem + kBar + 68, 256); tmem_relinquish(); }
    // A: row-major [128][slabs*128 B] -> swizzled slabs, written by the generic proxy
    for (int s = 0; s < slabs; ++s)
        for (int k = 0; k < 8; ++k)
            *reinterpret_cast<uint4*>(sm + s * 16384 + sw_off(row, k)) =
                *reinterpret_cast<const uint4*>(a + static_cast<size_t>(row) * slabs * 128 + s * 128 + k * 16);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(smem + kBar, w_stage * slabs);
        for (int s = 0; s < slabs; ++s) bulk_g2s(smem + kW + s * w_stage, w + s * w_stage, w_stage, smem + kBar);
        mbar_wait(smem + kBar, 0, abort_flag, kErrMmaWeights);
        tc_fence_after();
        const uint32_t idesc = mode == 0 ? umma_idesc(kAccS32, kFmtS8, kFmtS8, 128, 128)
                             : mode == 1 ? umma_idesc(kAccS32, kFmtU8, kFmtS8, 128, 128)
                             : mode == 2 ? umma_idesc(kAccS32, kFmtS8, kFmtS8, 128, 192)
                             : mode == 3 ? umma_idesc(kAccF32, kFmtF16, kFmtF16, 128, 96)
                                         : umma_idesc(kAccF32, kFmtE4M3, kFmtE4M3, 128, 128);
        for (int s = 0; s < slabs; ++s) {
            const uint64_t ad = umma_desc_k128(smem + s * 16384), bd = umma_desc_k128(smem + kW + s * w_stage);
            for (int k = 0; k < 4; ++k) {
                if (mode == 3)      umma_f16(tmem, ad + 2 * k, bd + 2 * k, idesc, (s | k) ? 1u : 0u);
                else if (mode == 4) umma_f8(tmem, ad + 2 * k, bd + 2 * k, idesc, (s | k) ? 1u : 0u);
                else                umma_i8(tmem, ad + 2 * k, bd + 2 * k, idesc, (s | k) ? 1u : 0u);
            }
        }
        tc_commit(smem + kBar + 8);
    }
    mbar_wait(smem + kBar + 8, 0, abort_flag, kErrRowAcc);
    tc_fence_after();
    for (int c0 = 0; c0 < n; c0 += 32) {
        uint32_t acc[32];
        tmem_ld32(tmem + (static_cast<uint32_t>(32 * warp) << 16) + c0, acc);
        tmem_wait_ld();
        for (int i = 0; i < 32; ++i) out[static_cast<size_t>(row) * n + c0 + i] = acc[i];
    }
    (void)lane;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tmem, 256);
    if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(status, 0, *abort_flag);
}

}  // namespace bf

// ==========================================================================================
// Host side: the C ABI.
// ==========================================================================================
namespace {

thread_local std::string g_err;

int fail(int code, const std::string& msg) {
    g_err = msg;
    return code;
}
#define BF_CUDA(call)                                                                      \
    do {                                                                                   \
        cudaError_t e_ = (call);                                                           \
        if (e_ != cudaSuccess)                                                             \
            return fail(BF_ECUDA, std::string(#call) + ": " + cudaGetErrorString(e_));    \
    } while (0)

// Makes `device` current for the scope of an entry point and puts the caller's device back on
// the way out, so that a call on cuda:1 does not leave a single-process multi-GPU program
// allocating and launching on cuda:1 afterwards.
struct DeviceScope {
    int prev = -1;
    cudaError_t err = cudaSuccess;
    explicit DeviceScope(int device) {
        err = cudaGetDevice(&prev);
        if (err == cudaSuccess && prev != device) err = cudaSetDevice(device);
        else if (err == cudaSuccess) prev = -1;          // already current: nothing to restore
    }
    ~DeviceScope() { if (prev >= 0) cudaSetDevice(prev); }
    DeviceScope(const DeviceScope&) = delete;
    DeviceScope& operator=(const DeviceScope&) = delete;
};
#define BF_ON_DEVICE(device)                                                                  \
    DeviceScope device_scope_(device);                                                        \
    if (device_scope_.err != cudaSuccess)                                                     \
        return fail(BF_ECUDA, std::string("selecting the device: ") + cudaGetErrorString(device_scope_.err))

struct BlobHeader {
    uint32_t magic, version, n_layers, n_value, vmode;
    float eps;
    uint32_t rj_mode, quant;      // quant: 3 = int8 all four matmuls, 1 = e4m3 FFN
    uint64_t off_w, bytes_w, off_lp, bytes_lp, off_emb, bytes_emb, off_tail, bytes_tail, off_rj, bytes_rj, total;
};

}  // namespace

struct bf_handle {
    int device = 0;
    BlobHeader hdr{};
    uint8_t* blob = nullptr;
    int* status = nullptr;
    unsigned long long* prof = nullptr;
    bool prof_on = false;
    bool rsqrt_rn = false;        // BF_OPT_RSQRT_RN
    int sm_count = 0;
    long long launches = 0;
    // staging for bf_forward_host
    int cap_n = 0;
    uint8_t* d_in = nullptr;      // boards | control | rep | legal
    uint8_t* d_out = nullptr;     // policy | promo | value
    cudaStream_t stream = nullptr;       // inputs and kernels of bf_forward_host
    cudaStream_t copy_stream = nullptr;  // its device-to-host copies
    cudaEvent_t chunk_done = nullptr;
    cudaEvent_t copy_t0 = nullptr, copy_t1 = nullptr;   // around the first copy-out of bf_forward_host
    double d2h_gbps = 0.0;        // what that copy last measured; 0 = not measured yet
    int host_plan = 0;            // BF_OPT_HOST_PLAN: 0 by the measured link, 1 fast-link sizes, 2 equal launches
    int one_board_factor = 1;     // BF_OPT_ONE_BOARD: batches up to this many boards per SM use the one-board form
};

namespace {

// Device staging of the host-buffer calls: inputs (boards, control, rep, legality words) and
// outputs (sized for the logits, the largest output set), grown to the largest n seen.
int ensure_staging(bf_handle* h, int n) {
    if (n <= h->cap_n) return BF_OK;
    cudaFree(h->d_in); cudaFree(h->d_out);
    h->d_in = h->d_out = nullptr; h->cap_n = 0;
    BF_CUDA(cudaMalloc(&h->d_in, static_cast<size_t>(n) * (64 + 2 + 1 + 256) + 1024));
    BF_CUDA(cudaMalloc(&h->d_out, static_cast<size_t>(n) * (4096 + 256 + 4) + 1024));
    h->cap_n = n;
    return BF_OK;
}

// The device-side alias of a pinned, mapped host allocation, or null for any other pointer.
void* mapped_host(const void* p) {
    if (p == nullptr) return nullptr;
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}

// bf_forward_host sizes its launches by how many times faster this GPU copies a position's logits
// to the host than it evaluates a position.
constexpr double kEvalGBps = 8.8;        // logits a B200 produces per second at full rate (4356 B x 2.03 M)
constexpr double kFastLinkRatio = 6.0;   // a GPU alone on its link: 55 GB/s against those 8.8

// The launch sizes of bf_forward_host for `n` positions on a GPU whose wave is `wave` positions:
// at most 16, in launch order, summing to n.  `gbps` is the measured copy rate (0: not known yet).
int host_plan_sizes(int n, int wave, int plan, double gbps, int* sizes, bool* slow) {
    // how many times faster this GPU copies a position out than it evaluates one
    double ratio = kFastLinkRatio;
    if (plan == 0 && gbps > 0.0) ratio = gbps / kEvalGBps;
    if (ratio > kFastLinkRatio) ratio = kFastLinkRatio;
    const bool slow_link = plan == 2 || ratio < 1.5;
    int n_chunks = 0;
    if (slow_link) {
        const int last = n < wave ? n : wave;
        const int rest = n - last;
        if (rest > 0) {
            int m = (rest + 2 * wave - 1) / (2 * wave);
            if (m > 14) m = 14;
            const int piece = ((rest + m - 1) / m + 3) & ~3;
            for (int left = rest; left > 0; left -= piece) sizes[n_chunks++] = left < piece ? left : piece;
        }
        sizes[n_chunks++] = last;
    } else {
        int rest = n, tmp[16], k = 0;
        double want = wave;
        while (rest > 0 && k < 15) {
            int m = static_cast<int>(want / wave) * wave;      // whole waves, rounded down: the margin
            if (m > rest || want >= 1e9) m = rest;
            tmp[k++] = m;
            rest -= m;
            want *= ratio;
        }
        if (rest > 0) tmp[k++] = rest;
        for (int i = k - 1; i >= 0; --i) sizes[n_chunks++] = tmp[i];          // largest first
    }
    if (slow != nullptr) *slow = slow_link;
    return n_chunks;
}

struct PriorOut {
    void* prior;
    int16_t* move;
    int* nedges;
    int e_cap;
};
struct Backbone {
    const void* x;              // device: activations in, [n,32,256] fp16
    const int8_t* alive;        // device: per-token alive flags [n,32] or null (all alive)
};
struct LeafList {
    const int* index;           // device: positions to evaluate, as places in the staged arrays
    const int* count;           // device: how many of them (read by the kernel when it starts)
};

int launch(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
           const uint64_t* legal, int n, void* policy, void* promo, float* value, void* y, int stage,
           int stage_layer, int cap_layer, int cap_op, uint8_t* cap_a, int32_t* cap_acc, cudaStream_t stream,
           const PriorOut* po = nullptr, const LeafList* leaves = nullptr, const Backbone* bb = nullptr) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (bb == nullptr && (boards == nullptr || control == nullptr || rep == nullptr))
        return fail(BF_EINVAL, "boards, control and rep must be non-null");
    BF_ON_DEVICE(h->device);
    bf::Params p{};
    p.boards = boards; p.control = control; p.rep = rep; p.legal = legal;
    p.n = n; p.n_layers = static_cast<int>(h->hdr.n_layers);
    p.n_value = static_cast<int>(h->hdr.n_value); p.vmode = static_cast<int>(h->hdr.vmode);
    p.quant = static_cast<int>(h->hdr.quant);
    p.rsqrt_rn = h->rsqrt_rn ? 1 : 0;
    p.eps = h->hdr.eps;
    p.one = 1.0f;
    p.wstream = h->blob + h->hdr.off_w;
    p.lparams = h->blob + h->hdr.off_lp;
    p.emb = reinterpret_cast<const __half*>(h->blob + h->hdr.off_emb);
    p.tail = reinterpret_cast<const __half*>(h->blob + h->hdr.off_tail);
    p.rj_mode = static_cast<int>(h->hdr.rj_mode);
    p.rj = p.rj_mode ? reinterpret_cast<const __half*>(h->blob + h->hdr.off_rj) : nullptr;
    p.policy = static_cast<__half*>(policy); p.promo = static_cast<__half*>(promo); p.value = value;
    p.y = static_cast<__half*>(y); p.debug_stage = stage; p.debug_layer = stage_layer;
    p.cap_layer = cap_layer; p.cap_op = cap_op; p.cap_a = cap_a; p.cap_acc = cap_acc;
    p.status = h->status;
    p.prof = h->prof_on ? h->prof : nullptr;
    if (po != nullptr) {
        p.prior = static_cast<__half*>(po->prior); p.move = po->move; p.nedges = po->nedges; p.e_cap = po->e_cap;
    }
    if (leaves != nullptr) { p.leaf_index = leaves->index; p.leaf_count = leaves->count; }
    if (bb != nullptr) { p.x_in = static_cast<const __half*>(bb->x); p.alive_in = bb->alive; }
    const int n_tiles = (n + 3) / 4;
    const int grid = n_tiles < h->sm_count ? n_tiles : h->sm_count;
    // the instrumented instantiation only when a dump, a capture or the phase clock is asked for
    const bool dbg = stage != 0 || cap_layer >= 0 || p.prof != nullptr;
    if (p.quant == 0) {
        if (cap_layer >= 0) return fail(BF_ENOTSUP, "operand capture is for the int8 arithmetic");
        if (p.rj_mode != 0) {
            if (dbg) bf::encoder_kernel<true, true, bf::kArF16><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
            else     bf::encoder_kernel<false, true, bf::kArF16><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        } else if (dbg) bf::encoder_kernel<true, false, bf::kArF16><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else     bf::encoder_kernel<false, false, bf::kArF16><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
    } else if (p.quant == 4) {
        if (cap_layer >= 0) return fail(BF_ENOTSUP, "operand capture is for the int8 arithmetic");
        if (dbg) bf::encoder_kernel<true, false, bf::kArI8Qkv><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else     bf::encoder_kernel<false, false, bf::kArI8Qkv><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
    } else if (p.quant == 2) {
        if (cap_layer >= 0) return fail(BF_ENOTSUP, "operand capture is for the int8 arithmetic");
        if (dbg) bf::encoder_kernel<true, false, bf::kArI8Ffn><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else     bf::encoder_kernel<false, false, bf::kArI8Ffn><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
    } else if (p.quant == 1) {
        if (cap_layer >= 0) return fail(BF_ENOTSUP, "operand capture is for the int8 arithmetic");
        if (dbg) bf::encoder_kernel<true, false, bf::kArE4M3><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else     bf::encoder_kernel<false, false, bf::kArE4M3><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
    } else if (p.rj_mode != 0) {
        if (dbg) bf::encoder_kernel<true, true, bf::kArInt8><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else     bf::encoder_kernel<false, true, bf::kArInt8><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
    } else {
        // a batch that leaves SMs idle (at most one board per SM) runs in the one-board-per-tile
        // form: sixteen row warps per board instead of four, about half the latency, same bits
        const bool small_form = !dbg && bb == nullptr && p.vmode != 2 && h->one_board_factor > 0;
        const bool one = small_form && n <= h->sm_count * h->one_board_factor;
        const int grid_one = n < h->sm_count ? n : h->sm_count;
        if (dbg) bf::encoder_kernel<true, false, bf::kArInt8><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else if (one)
            bf::encoder_kernel<false, false, bf::kArInt8, bf::kFormOne><<<grid_one, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else if (small_form && leaves != nullptr)
            // a leaf list may turn out short: one CTA per SM, and the kernel picks the form by the
            // count it reads
            bf::encoder_kernel<false, false, bf::kArInt8, bf::kFormByCount><<<grid_one, bf::kThreads, bf::kSmemRequest, stream>>>(p);
        else     bf::encoder_kernel<false, false, bf::kArInt8><<<grid, bf::kThreads, bf::kSmemRequest, stream>>>(p);
    }
    BF_CUDA(cudaGetLastError());
    h->launches++;
    return BF_OK;
}

}  // namespace

extern "C" {

const char* bf_version(void) { return "brokefish_b200 0.1 sm_100a"; }

const char* bf_last_error(void) { return g_err.c_str(); }

int bf_create(const void* blob, size_t blob_bytes, int device, bf_handle** out) {
    if (out == nullptr) return fail(BF_EINVAL, "out is null");
    *out = nullptr;
    if (blob == nullptr || blob_bytes < 256) return fail(BF_EINVAL, "blob is null or too small");
    BF_ON_DEVICE(device);
    BlobHeader hdr;
    BF_CUDA(cudaMemcpy(&hdr, blob, sizeof(hdr), cudaMemcpyDefault));
    if (hdr.magic != BF_BLOB_MAGIC) return fail(BF_EINVAL, "blob magic mismatch");
    if (hdr.version != BF_BLOB_VERSION) return fail(BF_EINVAL, "blob version mismatch");
    if (hdr.total != blob_bytes) return fail(BF_EINVAL, "blob size does not match its header");
    if (hdr.n_layers < 1 || hdr.n_layers > 64) return fail(BF_EINVAL, "n_layers out of range");
    if (hdr.quant > 4)
        return fail(BF_EINVAL, "blob arithmetic must be 3 (int8), 2 (int8 FFN only), 4 (int8 FFN and QKV), "
                               "1 (e4m3 FFN) or 0 (fp16)");
    if ((hdr.quant == 1 || hdr.quant == 2 || hdr.quant == 4) && hdr.rj_mode != 0)
        return fail(BF_ENOTSUP, "re-injection is built for the int8 and fp16 arithmetics, as in the reference");
    const uint64_t layer_stream = (hdr.quant == 1 || hdr.quant == 2) ? bf::Cfg<bf::kArE4M3>::kLayerStream
                                : hdr.quant == 4 ? bf::Cfg<bf::kArI8Qkv>::kLayerStream
                                : hdr.quant == 0 ? bf::Cfg<bf::kArF16>::kLayerStream
                                                 : bf::Cfg<bf::kArInt8>::kLayerStream;
    if (hdr.bytes_w != static_cast<uint64_t>(hdr.n_layers) * layer_stream + bf::kHeadStages * bf::kHeadStage ||
        hdr.bytes_lp != static_cast<uint64_t>(hdr.n_layers) * bf::kLparamStride ||
        hdr.bytes_emb != 184u * 256u * 2u || hdr.bytes_tail != bf::kTailBytes || hdr.rj_mode > 2 ||
        hdr.bytes_rj != (hdr.rj_mode ? static_cast<uint64_t>(hdr.n_layers) * hdr.rj_mode * 16u : 0u))
        return fail(BF_EINVAL, "blob section sizes do not match this build");
    if ((hdr.off_w | hdr.off_lp | hdr.off_emb | hdr.off_tail | hdr.off_rj) & 255u)
        return fail(BF_EINVAL, "blob sections must be 256-byte aligned");
    if (hdr.off_w + hdr.bytes_w > blob_bytes || hdr.off_lp + hdr.bytes_lp > blob_bytes ||
        hdr.off_emb + hdr.bytes_emb > blob_bytes || hdr.off_tail + hdr.bytes_tail > blob_bytes ||
        hdr.off_rj + hdr.bytes_rj > blob_bytes)
        return fail(BF_EINVAL, "blob section outside the blob");
    if (hdr.n_value != 1 && hdr.n_value != 3) return fail(BF_EINVAL, "n_value must be 1 or 3");
    if (hdr.vmode > 2) return fail(BF_EINVAL, "unknown value mode");
    cudaDeviceProp prop;
    BF_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(BF_ENOTSUP, "this library needs a compute capability 10.x (sm_100a) device");
    bf_handle* h = new (std::nothrow) bf_handle();
    if (h == nullptr) return fail(BF_EINVAL, "out of host memory");
    h->device = device; h->hdr = hdr; h->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaMalloc(&h->blob, blob_bytes);
    if (e == cudaSuccess) e = cudaMemcpy(h->blob, blob, blob_bytes, cudaMemcpyDefault);
    if (e == cudaSuccess) e = cudaMalloc(&h->status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(h->status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->copy_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&h->chunk_done, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreate(&h->copy_t0);
    if (e == cudaSuccess) e = cudaEventCreate(&h->copy_t1);
    const void* kernels[14] = {
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, false, bf::kArI8Qkv>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, false, bf::kArI8Qkv>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, false, bf::kArI8Ffn>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, false, bf::kArI8Ffn>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, true, bf::kArF16>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, true, bf::kArF16>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, false, bf::kArInt8>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, false, bf::kArInt8>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, true, bf::kArInt8>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, true, bf::kArInt8>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, false, bf::kArE4M3>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, false, bf::kArE4M3>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<false, false, bf::kArF16>),
        reinterpret_cast<const void*>(&bf::encoder_kernel<true, false, bf::kArF16>)};
    for (int i = 0; i < 14 && e == cudaSuccess; ++i)
        e = cudaFuncSetAttribute(kernels[i], cudaFuncAttributeMaxDynamicSharedMemorySize, bf::kSmemRequest);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(bf::encoder_kernel<false, false, bf::kArInt8, bf::kFormOne>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, bf::kSmemRequest);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(bf::encoder_kernel<false, false, bf::kArInt8, bf::kFormByCount>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, bf::kSmemRequest);
    if (e != cudaSuccess) {
        bf_destroy(h);
        return fail(BF_ECUDA, std::string("bf_create: ") + cudaGetErrorString(e));
    }
    *out = h;
    return BF_OK;
}

int bf_destroy(bf_handle* h) {
    if (h == nullptr) return BF_OK;
    DeviceScope device_scope_(h->device);
    if (h->stream) { cudaStreamSynchronize(h->stream); cudaStreamDestroy(h->stream); }
    if (h->copy_stream) { cudaStreamSynchronize(h->copy_stream); cudaStreamDestroy(h->copy_stream); }
    if (h->chunk_done) cudaEventDestroy(h->chunk_done);
    if (h->copy_t0) cudaEventDestroy(h->copy_t0);
    if (h->copy_t1) cudaEventDestroy(h->copy_t1);
    cudaFree(h->blob); cudaFree(h->status); cudaFree(h->prof); cudaFree(h->d_in); cudaFree(h->d_out);
    delete h;
    return BF_OK;
}

int bf_info(const bf_handle* h, int* n_layers, int* n_value, int* vmode) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (n_layers) *n_layers = static_cast<int>(h->hdr.n_layers);
    if (n_value) *n_value = static_cast<int>(h->hdr.n_value);
    if (vmode) *vmode = static_cast<int>(h->hdr.vmode);
    return BF_OK;
}

int bf_forward(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
               const uint64_t* legal, int n, void* policy, void* promo, float* value, void* stream) {
    return launch(h, boards, control, rep, legal, n, policy, promo, value, nullptr, 0, 0, -1, -1, nullptr,
                  nullptr, static_cast<cudaStream_t>(stream));
}

int bf_forward_priors(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                      const uint64_t* legal, int n, int e_cap, void* prior, int16_t* move, int* nedges,
                      float* value, void* policy, void* promo, void* stream) {
    if (prior == nullptr || move == nullptr || nedges == nullptr) return fail(BF_EINVAL, "prior, move and nedges must be non-null");
    if (e_cap < 1 || e_cap > 255) return fail(BF_EINVAL, "e_cap must be in 1..255");
    if (legal == nullptr && policy != nullptr)
        return fail(BF_EINVAL, "the masked policy needs the legality words; pass them or leave policy null");
    const PriorOut po{prior, move, nedges, e_cap};
    return launch(h, boards, control, rep, legal, n, policy, promo, value, nullptr, 0, 0, -1, -1, nullptr,
                  nullptr, static_cast<cudaStream_t>(stream), &po);
}

int bf_forward_leaves(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                      const uint64_t* legal, const int* leaf_index, const int* leaf_count, int capacity,
                      void* policy, void* promo, float* value, int e_cap, void* prior, int16_t* move,
                      int* nedges, void* stream) {
    if (leaf_index == nullptr || leaf_count == nullptr) return fail(BF_EINVAL, "leaf_index and leaf_count must be non-null");
    const bool priors = prior != nullptr || move != nullptr || nedges != nullptr;
    if (priors) {
        if (prior == nullptr || move == nullptr || nedges == nullptr)
            return fail(BF_EINVAL, "prior, move and nedges go together");
        if (e_cap < 1 || e_cap > 255) return fail(BF_EINVAL, "e_cap must be in 1..255");
        if (legal == nullptr && policy != nullptr)
            return fail(BF_EINVAL, "the masked policy needs the legality words; pass them or leave policy null");
    }
    const PriorOut po{prior, move, nedges, e_cap};
    const LeafList ll{leaf_index, leaf_count};
    return launch(h, boards, control, rep, legal, capacity, policy, promo, value, nullptr, 0, 0, -1, -1, nullptr,
                  nullptr, static_cast<cudaStream_t>(stream), priors ? &po : nullptr, &ll);
}

int bf_movegen(int device, const uint16_t* boards, const int16_t* control, int n, uint64_t* mask,
               unsigned char* in_check, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (boards == nullptr || control == nullptr || mask == nullptr)
        return fail(BF_EINVAL, "boards, control and mask must be non-null");
    BF_ON_DEVICE(device);
    bfmg::engine_board_kernel<false, false><<<(n + bfmg::kTpbThreads - 1) / bfmg::kTpbThreads, bfmg::kTpbThreads,
                                               bfmg::kTpbSmem, static_cast<cudaStream_t>(stream)>>>(
        boards, control, nullptr, nullptr, nullptr, n, nullptr, nullptr, nullptr,
        reinterpret_cast<unsigned long long*>(mask), in_check, nullptr, nullptr);
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_hash(int device, const uint16_t* boards, const int16_t* control, int n, uint64_t* hash, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (boards == nullptr || control == nullptr || hash == nullptr)
        return fail(BF_EINVAL, "boards, control and hash must be non-null");
    BF_ON_DEVICE(device);
    bfmg::engine_board_kernel<false, false><<<(n + bfmg::kTpbThreads - 1) / bfmg::kTpbThreads, bfmg::kTpbThreads,
                                               bfmg::kTpbSmem, static_cast<cudaStream_t>(stream)>>>(
        boards, control, nullptr, nullptr, nullptr, n, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
        reinterpret_cast<unsigned long long*>(hash));
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_history_push(int device, uint64_t* ring, long long* length, const uint64_t* hash,
                    const unsigned char* irreversible, int n, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (ring == nullptr || length == nullptr || hash == nullptr || irreversible == nullptr)
        return fail(BF_EINVAL, "ring, length, hash and irreversible must be non-null");
    BF_ON_DEVICE(device);
    bfmg::history_push_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<unsigned long long*>(ring), length, reinterpret_cast<const unsigned long long*>(hash),
        irreversible, n);
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_repetition_count(int device, const uint64_t* hash, const uint64_t* ring, const long long* length, int n,
                        int* count, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (ring == nullptr || length == nullptr || hash == nullptr || count == nullptr)
        return fail(BF_EINVAL, "hash, ring, length and count must be non-null");
    BF_ON_DEVICE(device);
    bfmg::repetition_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const unsigned long long*>(hash), reinterpret_cast<const unsigned long long*>(ring), length,
        n, count);
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_step(int device, const uint16_t* boards, const int16_t* control, const int* move,
            const signed char* promo, int n, uint16_t* boards_out, int16_t* control_out,
            unsigned char* irreversible, uint64_t* mask, unsigned char* in_check, uint64_t* hash, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (boards == nullptr || control == nullptr || move == nullptr || boards_out == nullptr || control_out == nullptr)
        return fail(BF_EINVAL, "boards, control, move, boards_out and control_out must be non-null");
    BF_ON_DEVICE(device);
    bfmg::engine_board_kernel<true, false><<<(n + bfmg::kTpbThreads - 1) / bfmg::kTpbThreads, bfmg::kTpbThreads,
                                              bfmg::kTpbSmem, static_cast<cudaStream_t>(stream)>>>(
        boards, control, move, promo, nullptr, n, boards_out, control_out, irreversible,
        reinterpret_cast<unsigned long long*>(mask), in_check, nullptr, reinterpret_cast<unsigned long long*>(hash));
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_terminal(int device, const uint64_t* mask, const unsigned char* in_check, const int16_t* control,
                const uint16_t* boards, const int* rep_count, int n, unsigned char* code, signed char* result,
                void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (mask == nullptr || in_check == nullptr || control == nullptr || boards == nullptr || code == nullptr)
        return fail(BF_EINVAL, "mask, in_check, control, boards and code must be non-null");
    BF_ON_DEVICE(device);
    bfmg::terminal_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const unsigned long long*>(mask), in_check, control, boards, rep_count, n, code, result);
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_random_ply(int device, uint16_t* boards, int16_t* control, uint64_t* mask, const float* r,
                  const signed char* promo, int n, int* move, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (boards == nullptr || control == nullptr || mask == nullptr || r == nullptr)
        return fail(BF_EINVAL, "boards, control, mask and r must be non-null");
    BF_ON_DEVICE(device);
    bfmg::engine_board_kernel<true, true><<<(n + bfmg::kTpbThreads - 1) / bfmg::kTpbThreads, bfmg::kTpbThreads,
                                             bfmg::kTpbSmem, static_cast<cudaStream_t>(stream)>>>(
        boards, control, nullptr, promo, r, n, boards, control, nullptr,
        reinterpret_cast<unsigned long long*>(mask), nullptr, move, nullptr);
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

void bf_int8_q_max(int* signed_max, int* unsigned_max) {
    if (signed_max != nullptr) *signed_max = static_cast<int>(bf::kQMaxS8);
    if (unsigned_max != nullptr) *unsigned_max = static_cast<int>(bf::kQMaxU8);
}
double bf_fp8_q_max(void) { return static_cast<double>(bf::kQMaxE4M3); }

int bf_forward_backbone(bf_handle* h, const void* x, const int8_t* alive, int n, void* y, void* stream) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (n == 0) return BF_OK;
    if (x == nullptr || y == nullptr) return fail(BF_EINVAL, "x and y must be non-null");
    if (h->hdr.quant != 0)
        return fail(BF_ENOTSUP, "the backbone-only entry runs the fp16 arithmetic only, as the reference's does");
    const Backbone bb{x, alive};
    // the residual stream at the end of the last layer, through the instrumented arm's dump
    return launch(h, nullptr, nullptr, nullptr, nullptr, n, nullptr, nullptr, nullptr, y, 10,
                  static_cast<int>(h->hdr.n_layers) - 1, -1, -1, nullptr, nullptr,
                  static_cast<cudaStream_t>(stream), nullptr, nullptr, &bb);
}

int bf_forward_stage_at(bf_handle* h, const uint16_t* boards, const int16_t* control,
                        const uint8_t* rep, int n, int layer, int stage, void* y, void* stream) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (y == nullptr) return fail(BF_EINVAL, "y is null");
    if (!((stage >= 1 && stage <= 10))) return fail(BF_EINVAL, "unknown stage");
    if (layer < 0 || layer >= static_cast<int>(h->hdr.n_layers)) return fail(BF_EINVAL, "layer out of range");
    return launch(h, boards, control, rep, nullptr, n, nullptr, nullptr, nullptr, y, stage, layer, -1, -1,
                  nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

int bf_forward_stage(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                     int n, int stage, void* y, void* stream) {
    if (!(stage == 9 || (stage >= 1 && stage <= 8))) return fail(BF_EINVAL, "unknown stage");
    return bf_forward_stage_at(h, boards, control, rep, n, 0, stage, y, stream);
}

int bf_forward_capture(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                       int n, int layer, int op, uint8_t* a_bytes, int32_t* acc, void* stream) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (a_bytes == nullptr || acc == nullptr) return fail(BF_EINVAL, "capture buffers are null");
    if (layer < 0 || layer >= static_cast<int>(h->hdr.n_layers)) return fail(BF_EINVAL, "layer out of range");
    if (op < BF_OP_QKV || op > BF_OP_FF2 + 3) return fail(BF_EINVAL, "unknown op");
    return launch(h, boards, control, rep, nullptr, n, nullptr, nullptr, nullptr, nullptr, 0, 0, layer, op,
                  a_bytes, acc, static_cast<cudaStream_t>(stream));
}

int bf_forward_host(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                    const uint64_t* legal, int n, void* policy, void* promo, float* value) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (boards == nullptr || control == nullptr || rep == nullptr)
        return fail(BF_EINVAL, "boards, control and rep must be non-null");
    BF_ON_DEVICE(h->device);
    { const int rc = ensure_staging(h, n); if (rc != BF_OK) return rc; }
    const size_t N = static_cast<size_t>(h->cap_n);
    uint8_t* d_legal = h->d_in;                         // 8-byte aligned first
    uint8_t* d_boards = d_legal + N * 256;
    uint8_t* d_control = d_boards + N * 64;
    uint8_t* d_rep = d_control + N * 2;
    uint8_t* d_policy = h->d_out;
    uint8_t* d_promo = d_policy + N * 4096;
    uint8_t* d_value = d_promo + N * 256;
    cudaStream_t s = h->stream;
    BF_CUDA(cudaMemcpyAsync(d_boards, boards, static_cast<size_t>(n) * 64, cudaMemcpyHostToDevice, s));
    BF_CUDA(cudaMemcpyAsync(d_control, control, static_cast<size_t>(n) * 2, cudaMemcpyHostToDevice, s));
    BF_CUDA(cudaMemcpyAsync(d_rep, rep, static_cast<size_t>(n), cudaMemcpyHostToDevice, s));
    if (legal) BF_CUDA(cudaMemcpyAsync(d_legal, legal, static_cast<size_t>(n) * 256, cudaMemcpyHostToDevice, s));
    // The batch goes out as a few launches so that the copy-out of a finished launch overlaps the
    // next launch's compute on a second stream and only the last launch's copy is exposed.  Which
    // plan is best depends on how fast this GPU reaches host memory right now, which the call
    // measures on its largest copy and averages over the calls (measured on 8-GPU B200 boxes: 55 GB/s
    // for one GPU alone, 12-19 GB/s each when eight GPUs copy at once; evaluating produces 8.8 GB/s).
    // With r = copy rate / evaluation rate:
    //   r >= 1.5    launches of shrinking size, largest first, the last one a single wave (one
    //               tile per SM), each launch r times the one after it (in whole waves, rounded
    //               down) so that its copy hides behind the next launch; r is capped at 6, a GPU
    //               alone on its link: [3504, 592] positions for a batch of 4096.  Large launches
    //               keep the kernel's tile-to-tile pipelining.
    //   r < 1.5     equal launches of about two waves, so that every copy hides behind the next
    //               launch as long as copying is not slower than evaluating, and the last wave
    //               writes its logits straight into the caller's buffers when these are pinned
    //               and device-mapped: the link is the bottleneck then, and stores that cross it
    //               while the wave computes beat a copy that starts when the wave has ended.
    // (Everything through mapped memory was measured 10 % slower on a fast link -- the stores back
    // up behind the bus -- and the last wave alone 4 % slower than copying it.)
    const int wave = h->sm_count * 4;
    void* m_policy = mapped_host(policy);
    void* m_promo = mapped_host(promo);
    void* m_value = mapped_host(value);
    const bool all_mapped = policy != nullptr && promo != nullptr && value != nullptr &&
                            m_policy != nullptr && m_promo != nullptr && m_value != nullptr;
    cudaStream_t c = h->copy_stream;
    size_t timed_bytes = 0;
    auto copy_out = [&](int lo, int m, bool timed) -> int {
        const size_t o = static_cast<size_t>(lo), M = static_cast<size_t>(m);
        if (timed) BF_CUDA(cudaEventRecord(h->copy_t0, c));
        if (policy) BF_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(policy) + o * 4096, d_policy + o * 4096, M * 4096, cudaMemcpyDeviceToHost, c));
        if (timed) { BF_CUDA(cudaEventRecord(h->copy_t1, c)); timed_bytes = M * 4096; }
        if (promo) BF_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(promo) + o * 256, d_promo + o * 256, M * 256, cudaMemcpyDeviceToHost, c));
        if (value) BF_CUDA(cudaMemcpyAsync(value + o, d_value + o * 4, M * 4, cudaMemcpyDeviceToHost, c));
        return BF_OK;
    };
    int sizes[16];
    bool slow_link = false;
    const int n_chunks = host_plan_sizes(n, wave, h->host_plan, h->d2h_gbps, sizes, &slow_link);
    const bool direct_last = slow_link && all_mapped;
    int lo = 0, k_timed = 0;
    for (int k = 1; k < n_chunks; ++k)
        if (sizes[k] > sizes[k_timed]) k_timed = k;
    for (int k = 0; k < n_chunks; lo += sizes[k], ++k) {
        const int m = sizes[k];
        const size_t o = static_cast<size_t>(lo);
        const bool direct = direct_last && k == n_chunks - 1;
        int rc = launch(h, reinterpret_cast<uint16_t*>(d_boards) + o * 32, reinterpret_cast<int16_t*>(d_control) + o,
                        d_rep + o, legal ? reinterpret_cast<uint64_t*>(d_legal) + o * 32 : nullptr, m,
                        direct ? static_cast<uint8_t*>(m_policy) + o * 4096 : d_policy + o * 4096,
                        direct ? static_cast<uint8_t*>(m_promo) + o * 256 : d_promo + o * 256,
                        direct ? static_cast<float*>(m_value) + o : reinterpret_cast<float*>(d_value) + o, nullptr,
                        0, 0, -1, -1, nullptr, nullptr, s);
        if (rc != BF_OK) return rc;
        if (direct) break;
        BF_CUDA(cudaEventRecord(h->chunk_done, s));
        BF_CUDA(cudaStreamWaitEvent(c, h->chunk_done, 0));
        // the largest launch's copy is the link measurement (large enough to mean something)
        rc = copy_out(lo, m, k == k_timed && policy != nullptr && static_cast<size_t>(m) * 4096 >= (1u << 20));
        if (rc != BF_OK) return rc;
    }
    BF_CUDA(cudaStreamSynchronize(s));
    BF_CUDA(cudaStreamSynchronize(c));
    if (timed_bytes != 0) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, h->copy_t0, h->copy_t1) == cudaSuccess && ms > 0.f) {
            // averaged over the calls: with several GPUs on one link the rate a copy sees depends
            // on the sizes the other GPUs chose, which depend on the rates they saw
            const double now = static_cast<double>(timed_bytes) / (ms * 1e-3) / 1e9;
            h->d2h_gbps = h->d2h_gbps > 0.0 ? 0.5 * (h->d2h_gbps + now) : now;
        }
        else
            cudaGetLastError();
    }
    return BF_OK;
}

int bf_forward_priors_host(bf_handle* h, const uint16_t* boards, const int16_t* control, const uint8_t* rep,
                           const uint64_t* legal, int n, int e_cap, void* prior, int16_t* move, int* nedges,
                           float* value) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n == 0) return BF_OK;
    if (boards == nullptr || control == nullptr || rep == nullptr || legal == nullptr)
        return fail(BF_EINVAL, "boards, control, rep and legal must be non-null");
    if (prior == nullptr || move == nullptr || nedges == nullptr) return fail(BF_EINVAL, "prior, move and nedges must be non-null");
    if (e_cap < 1 || e_cap > 255) return fail(BF_EINVAL, "e_cap must be in 1..255");
    BF_ON_DEVICE(h->device);
    { const int rc = ensure_staging(h, n); if (rc != BF_OK) return rc; }
    const size_t N = static_cast<size_t>(h->cap_n), E = static_cast<size_t>(e_cap);
    uint8_t* d_legal = h->d_in;
    uint8_t* d_boards = d_legal + N * 256;
    uint8_t* d_control = d_boards + N * 64;
    uint8_t* d_rep = d_control + N * 2;
    // the output staging (sized for the logits) holds the much smaller edge lists
    uint8_t* d_nedges = h->d_out;
    uint8_t* d_value = d_nedges + N * 4;
    uint8_t* d_prior = d_value + N * 4;
    uint8_t* d_move = d_prior + N * E * 2;
    cudaStream_t s = h->stream, c = h->copy_stream;
    BF_CUDA(cudaMemcpyAsync(d_boards, boards, static_cast<size_t>(n) * 64, cudaMemcpyHostToDevice, s));
    BF_CUDA(cudaMemcpyAsync(d_control, control, static_cast<size_t>(n) * 2, cudaMemcpyHostToDevice, s));
    BF_CUDA(cudaMemcpyAsync(d_rep, rep, static_cast<size_t>(n), cudaMemcpyHostToDevice, s));
    BF_CUDA(cudaMemcpyAsync(d_legal, legal, static_cast<size_t>(n) * 256, cudaMemcpyHostToDevice, s));
    {
        // pinned, mapped outputs: the edge lists are small (392 B per position at e_cap 96), so
        // one launch writes them across the bus as it goes (measured 2 % faster than staging)
        void* m_prior = mapped_host(prior);
        void* m_move = mapped_host(move);
        void* m_ne = mapped_host(nedges);
        void* m_value = mapped_host(value);
        if (m_prior && m_move && m_ne && (value == nullptr || m_value)) {
            const PriorOut po{m_prior, static_cast<int16_t*>(m_move), static_cast<int*>(m_ne), e_cap};
            int rc = launch(h, reinterpret_cast<uint16_t*>(d_boards), reinterpret_cast<int16_t*>(d_control), d_rep,
                            reinterpret_cast<uint64_t*>(d_legal), n, nullptr, nullptr, static_cast<float*>(m_value),
                            nullptr, 0, 0, -1, -1, nullptr, nullptr, s, &po);
            if (rc != BF_OK) return rc;
            BF_CUDA(cudaStreamSynchronize(s));
            return BF_OK;
        }
    }
    const int wave = h->sm_count * 4;
    for (int lo = 0; lo < n; lo += wave) {
        const int m = n - lo < wave ? n - lo : wave;
        const size_t o = static_cast<size_t>(lo), M = static_cast<size_t>(m);
        const PriorOut po{d_prior + o * E * 2, reinterpret_cast<int16_t*>(d_move + o * E * 2),
                          reinterpret_cast<int*>(d_nedges) + o, e_cap};
        int rc = launch(h, reinterpret_cast<uint16_t*>(d_boards) + o * 32, reinterpret_cast<int16_t*>(d_control) + o,
                        d_rep + o, reinterpret_cast<uint64_t*>(d_legal) + o * 32, m, nullptr, nullptr,
                        reinterpret_cast<float*>(d_value) + o, nullptr, 0, 0, -1, -1, nullptr, nullptr, s, &po);
        if (rc != BF_OK) return rc;
        BF_CUDA(cudaEventRecord(h->chunk_done, s));
        BF_CUDA(cudaStreamWaitEvent(c, h->chunk_done, 0));
        BF_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(prior) + o * E * 2, d_prior + o * E * 2, M * E * 2, cudaMemcpyDeviceToHost, c));
        BF_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(move) + o * E * 2, d_move + o * E * 2, M * E * 2, cudaMemcpyDeviceToHost, c));
        BF_CUDA(cudaMemcpyAsync(nedges + o, d_nedges + o * 4, M * 4, cudaMemcpyDeviceToHost, c));
        if (value) BF_CUDA(cudaMemcpyAsync(value + o, d_value + o * 4, M * 4, cudaMemcpyDeviceToHost, c));
    }
    BF_CUDA(cudaStreamSynchronize(s));
    BF_CUDA(cudaStreamSynchronize(c));
    return BF_OK;
}

int bf_set_option(bf_handle* h, int option, int value) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    if (option == BF_OPT_RSQRT_RN) { h->rsqrt_rn = value != 0; return BF_OK; }
    if (option == BF_OPT_ONE_BOARD) {
        if (value < 0 || value > 8) return fail(BF_EINVAL, "BF_OPT_ONE_BOARD takes 0..8");
        h->one_board_factor = value;
        return BF_OK;
    }
    if (option == BF_OPT_HOST_PLAN) {
        if (value < 0 || value > 2) return fail(BF_EINVAL, "BF_OPT_HOST_PLAN takes 0, 1 or 2");
        h->host_plan = value;
        return BF_OK;
    }
    return fail(BF_EINVAL, "unknown option");
}

int bf_status(bf_handle* h, int* status) {
    if (h == nullptr || status == nullptr) return fail(BF_EINVAL, "null argument");
    BF_ON_DEVICE(h->device);
    BF_CUDA(cudaDeviceSynchronize());
    BF_CUDA(cudaMemcpy(status, h->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) {
        BF_CUDA(cudaMemset(h->status, 0, sizeof(int)));
        return fail(BF_EDEVICE, "a device-side bounded wait ran out (code " + std::to_string(*status) + ")");
    }
    return BF_OK;
}

long long bf_launch_count(const bf_handle* h) { return h ? h->launches : 0; }

double bf_host_link_gbps(const bf_handle* h) { return h ? h->d2h_gbps : 0.0; }

int bf_host_plan(int n, int sm_count, int plan, double gbps, int* sizes) {
    if (n < 1 || sm_count < 1 || plan < 0 || plan > 2 || sizes == nullptr)
        return fail(BF_EINVAL, "bf_host_plan: n and sm_count must be positive, plan 0..2, sizes non-null");
    return host_plan_sizes(n, sm_count * 4, plan, gbps, sizes, nullptr);
}

int bf_profile(bf_handle* h, int enable) {
    if (h == nullptr) return fail(BF_EINVAL, "null handle");
    BF_ON_DEVICE(h->device);
    if (enable && h->prof == nullptr) BF_CUDA(cudaMalloc(&h->prof, 16 * sizeof(unsigned long long)));
    if (h->prof != nullptr) BF_CUDA(cudaMemset(h->prof, 0, 16 * sizeof(unsigned long long)));
    h->prof_on = enable != 0;
    return BF_OK;
}

int bf_profile_read(bf_handle* h, long long* cycles, int n) {
    if (h == nullptr || cycles == nullptr || n < 0) return fail(BF_EINVAL, "bad argument");
    if (h->prof == nullptr) return fail(BF_EINVAL, "profiling was never enabled on this handle");
    BF_ON_DEVICE(h->device);
    BF_CUDA(cudaDeviceSynchronize());
    unsigned long long tmp[16];
    BF_CUDA(cudaMemcpy(tmp, h->prof, sizeof(tmp), cudaMemcpyDeviceToHost));
    BF_CUDA(cudaMemset(h->prof, 0, sizeof(tmp)));
    for (int i = 0; i < n && i < 16; ++i) cycles[i] = static_cast<long long>(tmp[i]);
    return BF_OK;
}

const char* bf_profile_phases(void) {
    return "embed,layernorm_quantise,wait_mma_qkv,qkv_epilogue,pair_barrier,attention,attn_readback,"
           "attn_quantise,out_proj_epilogue,ff1_epilogue,ff2_epilogue,heads,wait_mma_out,wait_mma_ff1,"
           "wait_mma_ff2,wait_mma_ff1_first";
}

int bf_measure_i8_peak(int device, int iters, double* tops, double* ms) {
    if (tops == nullptr || iters < 2 || iters > (1 << 22)) return fail(BF_EINVAL, "tops is null or iters out of range");
    BF_ON_DEVICE(device);
    cudaDeviceProp prop;
    BF_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(BF_ENOTSUP, "this library needs a compute capability 10.x (sm_100a) device");
    constexpr int kSmem = 49152 + 256 + 1024;
    BF_CUDA(cudaFuncSetAttribute(bf::i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    int* status = nullptr;
    BF_CUDA(cudaMalloc(&status, sizeof(int)));
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaError_t e = cudaMemset(status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    float best = 0.f;
    int st = 0;
    for (int rep = 0; rep < 4 && e == cudaSuccess; ++rep) {      // first repetition warms up
        cudaEventRecord(e0);
        bf::i8_peak_kernel<<<prop.multiProcessorCount, 128, kSmem>>>(iters, status);
        cudaEventRecord(e1);
        e = cudaEventSynchronize(e1);
        float t = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, e0, e1);
        if (rep > 0 && (best == 0.f || t < best)) best = t;
    }
    if (e == cudaSuccess) e = cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(status);
    if (e != cudaSuccess) return fail(BF_ECUDA, cudaGetErrorString(e));
    if (st != 0) return fail(BF_EDEVICE, "the probe's bounded wait ran out");
    const double ops = 2.0 * 128 * 256 * 32 * 4.0 * iters * prop.multiProcessorCount;
    *tops = ops / (best * 1e-3) / 1e12;
    if (ms != nullptr) *ms = best;
    return BF_OK;
}

int bf_measure_elementwise(int device, int block, int iters, double* elements_per_s, double* ms) {
    if (elements_per_s == nullptr || iters < 1 || iters > (1 << 22) || block < 0 || block > 11)
        return fail(BF_EINVAL, "elements_per_s is null, block not in 0..11 or iters out of range");
    BF_ON_DEVICE(device);
    cudaDeviceProp prop;
    BF_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) return fail(BF_ENOTSUP, "this library needs a compute capability 10.x (sm_100a) device");
    using Kernel = void (*)(const __half*, float, float, float, int, float*);
    static const Kernel kernels[12] = {bf::elementwise_probe_kernel<0, 512>, bf::elementwise_probe_kernel<1, 512>,
                                       bf::elementwise_probe_kernel<2, 512>, bf::elementwise_probe_kernel<3, 512>,
                                       bf::elementwise_probe_kernel<4, 512>, bf::elementwise_probe_kernel<5, 512>,
                                       bf::elementwise_probe_kernel<0, 256>, bf::elementwise_probe_kernel<0, 1024>,
                                       bf::elementwise_probe_kernel<8, 512>, bf::elementwise_probe_kernel<9, 512>,
                                       bf::elementwise_probe_kernel<10, 512>, bf::elementwise_probe_kernel<11, 512>};
    const int threads = block == 6 ? 256 : (block == 7 ? 1024 : 512);
    const int kSmem = 32 * threads * 4;
    BF_CUDA(cudaFuncSetAttribute(kernels[block], cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    const int sms = prop.multiProcessorCount;
    __half* bias = nullptr;
    float* out = nullptr;
    BF_CUDA(cudaMalloc(&bias, 256));
    cudaError_t e = cudaMalloc(&out, static_cast<size_t>(sms) * threads * sizeof(float));
    if (e == cudaSuccess) e = cudaMemset(bias, 0, 256);
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (e == cudaSuccess) e = cudaEventCreate(&e0);
    if (e == cudaSuccess) e = cudaEventCreate(&e1);
    float best = 0.f;
    for (int rep = 0; rep < 4 && e == cudaSuccess; ++rep) {      // first repetition warms up
        cudaEventRecord(e0);
        kernels[block]<<<sms, threads, kSmem>>>(bias, 0.01f, 0.02f, 1.0f, iters, out);
        cudaEventRecord(e1);
        e = cudaEventSynchronize(e1);
        float t = 0.f;
        if (e == cudaSuccess) e = cudaEventElapsedTime(&t, e0, e1);
        if (rep > 0 && (best == 0.f || t < best)) best = t;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(bias);
    if (out) cudaFree(out);
    if (e != cudaSuccess) return fail(BF_ECUDA, cudaGetErrorString(e));
    *elements_per_s = 32.0 * threads * iters * sms / (best * 1e-3);
    if (ms != nullptr) *ms = best;
    return BF_OK;
}

int bf_selftest_timeout(int device, int code, int* status, long long* waited_cycles) {
    if (status == nullptr || code < 1 || code > 99) return fail(BF_EINVAL, "status is null or code not in 1..99");
    BF_ON_DEVICE(device);
    int* d_status = nullptr;
    long long* d_waited = nullptr;
    BF_CUDA(cudaMalloc(&d_status, sizeof(int)));
    cudaError_t e = cudaMalloc(&d_waited, 2 * sizeof(long long));
    if (e == cudaSuccess) e = cudaMemset(d_status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(d_waited, 0, 2 * sizeof(long long));
    if (e == cudaSuccess) {
        bf::timeout_kernel<<<1, 64>>>(code, d_status, d_waited);
        e = cudaDeviceSynchronize();
    }
    long long w[2] = {0, 0};
    if (e == cudaSuccess) e = cudaMemcpy(status, d_status, sizeof(int), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemcpy(w, d_waited, sizeof(w), cudaMemcpyDeviceToHost);
    cudaFree(d_status);
    cudaFree(d_waited);
    if (e != cudaSuccess) return fail(BF_ECUDA, cudaGetErrorString(e));
    if (waited_cycles != nullptr) { waited_cycles[0] = w[0]; waited_cycles[1] = w[1]; }
    return BF_OK;
}

int bf_selftest_umma(int device, int mode, const void* a, const void* w_image, void* out) {
    if (mode < 0 || mode > 4 || a == nullptr || w_image == nullptr || out == nullptr)
        return fail(BF_EINVAL, "bad self-test argument");
    BF_ON_DEVICE(device);
    int* status = nullptr;
    BF_CUDA(cudaMalloc(&status, sizeof(int)));
    BF_CUDA(cudaMemset(status, 0, sizeof(int)));
    constexpr int kSmem = 163840 + 128 + 1024;
    BF_CUDA(cudaFuncSetAttribute(bf::selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
    bf::selftest_kernel<<<1, 128, kSmem>>>(mode, static_cast<const uint8_t*>(a),
                                           static_cast<const uint8_t*>(w_image),
                                           static_cast<uint32_t*>(out), status);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    int st = 0;
    if (e == cudaSuccess) e = cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(status);
    if (e != cudaSuccess) return fail(BF_ECUDA, std::string("self test: ") + cudaGetErrorString(e));
    if (st != 0) return fail(BF_EDEVICE, "self test: a bounded wait ran out (code " + std::to_string(st) + ")");
    return BF_OK;
}

}  // extern "C"

// ==========================================================================================
// An entry point that allocates nothing.
//
// Who this is for: code that may enqueue work on a GPU but must not grow its memory
// footprint while doing so -- a search worker running inside a process whose device memory
// was carved up in advance by somebody else, a plugin loaded into a host that forbids device
// allocation after start-up, a caller that runs with the allocator locked down for
// determinism.  Such a caller cannot create a `bf_handle` (bf_create calls cudaMalloc for the
// weight copy and the status word).  Here the caller keeps the packed weight blob in device
// memory it already owns and passes it on every call together with its inputs and outputs;
// the only memory the kernel needs beyond those -- its status word -- lives in a fixed
// 256-byte array that is part of the library image on every GPU that loads it.
// ==========================================================================================
namespace bf {
constexpr int kNoAllocScratchBytes = 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace bf

namespace {
constexpr int kNoAllocMaxDevices = 64;
struct NoAllocDevice {
    bool ready = false;
    void* scratch = nullptr;      // device address of bf::g_noalloc_scratch on this device
    int sm_count = 0;
    const void* blob = nullptr;   // blob whose header is cached below
    size_t blob_bytes = 0;
    BlobHeader hdr{};
};
NoAllocDevice g_noalloc[kNoAllocMaxDevices];
// One lock for the per-device records: set-up, the header cache and its reads.  A call holds it
// only while it looks the header up (and, for a blob it has not seen, reads it from the device),
// never across the launch.
std::mutex g_noalloc_mutex;

// Once per device, with that device current and the lock held: resolve the scratch array's
// device address (in host code the array's name is only a handle, never an address a kernel may
// use), raise the kernel's shared-memory limit, read the SM count, zero the scratch.
int noalloc_setup(int device, NoAllocDevice** out) {
    if (device < 0 || device >= kNoAllocMaxDevices) return fail(BF_EINVAL, "device index out of range");
    NoAllocDevice& d = g_noalloc[device];
    if (!d.ready) {
        cudaDeviceProp prop;
        BF_CUDA(cudaGetDeviceProperties(&prop, device));
        if (prop.major != 10)
            return fail(BF_ENOTSUP, "this library needs a compute capability 10.x (sm_100a) device");
        void* ptr = nullptr;
        BF_CUDA(cudaGetSymbolAddress(&ptr, bf::g_noalloc_scratch));
        BF_CUDA(cudaMemset(ptr, 0, bf::kNoAllocScratchBytes));
        BF_CUDA(cudaFuncSetAttribute(bf::encoder_kernel<false, false, bf::kArInt8>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     bf::kSmemRequest));
        d.scratch = ptr;
        d.sm_count = prop.multiProcessorCount;
        d.ready = true;
    }
    *out = &d;
    return BF_OK;
}

// The header of `blob_dev`, from the device's cache or read and checked now.  Returns a COPY, so
// that the launch below never reads a record another thread may be replacing.
int noalloc_header(NoAllocDevice* d, const void* blob_dev, size_t blob_bytes, BlobHeader* out) {
    if (d->blob != blob_dev || d->blob_bytes != blob_bytes) {
        BlobHeader hdr;
        BF_CUDA(cudaMemcpy(&hdr, blob_dev, sizeof(hdr), cudaMemcpyDeviceToHost));
        if (hdr.magic != BF_BLOB_MAGIC || hdr.version != BF_BLOB_VERSION || hdr.total != blob_bytes)
            return fail(BF_EINVAL, "blob header does not match (magic, version or size)");
        if (hdr.quant != 3)
            return fail(BF_ENOTSUP, "bf_forward_noalloc runs int8 \"all\" blobs (quant 3) only; this blob carries "
                                    "arithmetic " + std::to_string(hdr.quant) + ": use a handle (bf_create)");
        if (hdr.rj_mode != 0)
            return fail(BF_ENOTSUP, "bf_forward_noalloc does not run re-injecting networks: use a handle (bf_create)");
        if (hdr.n_layers < 1 || hdr.n_layers > 64 ||
            hdr.bytes_w != static_cast<uint64_t>(hdr.n_layers) * bf::Cfg<bf::kArInt8>::kLayerStream +
                               bf::kHeadStages * bf::kHeadStage ||
            hdr.bytes_lp != static_cast<uint64_t>(hdr.n_layers) * bf::kLparamStride ||
            hdr.bytes_emb != 184u * 256u * 2u || hdr.bytes_tail != bf::kTailBytes ||
            ((hdr.off_w | hdr.off_lp | hdr.off_emb | hdr.off_tail) & 255u) ||
            hdr.off_w + hdr.bytes_w > blob_bytes || hdr.off_lp + hdr.bytes_lp > blob_bytes ||
            hdr.off_emb + hdr.bytes_emb > blob_bytes || hdr.off_tail + hdr.bytes_tail > blob_bytes)
            return fail(BF_EINVAL, "blob sections do not match this build");
        if ((hdr.n_value != 1 && hdr.n_value != 3) || hdr.vmode > 2)
            return fail(BF_EINVAL, "n_value must be 1 or 3 and the value mode 0, 1 or 2");
        if (reinterpret_cast<uintptr_t>(blob_dev) & 255u)
            return fail(BF_EINVAL, "the device blob must be 256-byte aligned");
        d->hdr = hdr; d->blob = blob_dev; d->blob_bytes = blob_bytes;
    }
    *out = d->hdr;
    return BF_OK;
}
}  // namespace

extern "C" {

int bf_forward_noalloc(int device, const void* blob_dev, size_t blob_bytes, const uint16_t* boards,
                       const int16_t* control, const uint8_t* rep, const uint64_t* legal, int n,
                       void* policy, void* promo, float* value, void* stream) {
    if (n < 0) return fail(BF_EINVAL, "n must be >= 0");
    if (n > BF_NOALLOC_MAX_POSITIONS)
        return fail(BF_EINVAL, "bf_forward_noalloc: n exceeds BF_NOALLOC_MAX_POSITIONS (" +
                                   std::to_string(BF_NOALLOC_MAX_POSITIONS) + "); split the batch");
    if (blob_dev == nullptr || blob_bytes < 256) return fail(BF_EINVAL, "blob is null or too small");
    if (n > 0 && (boards == nullptr || control == nullptr || rep == nullptr))
        return fail(BF_EINVAL, "boards, control and rep must be non-null");
    if (device < 0 || device >= kNoAllocMaxDevices) return fail(BF_EINVAL, "device index out of range");
    BF_ON_DEVICE(device);
    BlobHeader hdr;
    void* scratch = nullptr;
    int sm_count = 0;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        NoAllocDevice* d = nullptr;
        int rc = noalloc_setup(device, &d);
        if (rc == BF_OK) rc = noalloc_header(d, blob_dev, blob_bytes, &hdr);
        if (rc != BF_OK) return rc;
        scratch = d->scratch;
        sm_count = d->sm_count;
    }
    if (n == 0) return BF_OK;
    const uint8_t* base = static_cast<const uint8_t*>(blob_dev);
    bf::Params p{};
    p.boards = boards; p.control = control; p.rep = rep; p.legal = legal;
    p.n = n; p.n_layers = static_cast<int>(hdr.n_layers);
    p.n_value = static_cast<int>(hdr.n_value); p.vmode = static_cast<int>(hdr.vmode);
    p.quant = 3;
    p.eps = hdr.eps;
    p.one = 1.0f;
    p.wstream = base + hdr.off_w;
    p.lparams = base + hdr.off_lp;
    p.emb = reinterpret_cast<const __half*>(base + hdr.off_emb);
    p.tail = reinterpret_cast<const __half*>(base + hdr.off_tail);
    p.rj = nullptr; p.rj_mode = 0;
    p.policy = static_cast<__half*>(policy); p.promo = static_cast<__half*>(promo); p.value = value;
    p.y = nullptr; p.debug_stage = 0; p.debug_layer = 0;
    p.cap_layer = -1; p.cap_op = -1; p.cap_a = nullptr; p.cap_acc = nullptr;
    p.status = static_cast<int*>(scratch);         // the device address, not the symbol
    p.prof = nullptr;
    const int n_tiles = (n + 3) / 4;
    const int grid = n_tiles < sm_count ? n_tiles : sm_count;
    bf::encoder_kernel<false, false, bf::kArInt8><<<grid, bf::kThreads, bf::kSmemRequest, static_cast<cudaStream_t>(stream)>>>(p);
    BF_CUDA(cudaGetLastError());
    return BF_OK;
}

int bf_noalloc_forget(int device) {
    if (device < 0 || device >= kNoAllocMaxDevices) return fail(BF_EINVAL, "device index out of range");
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    g_noalloc[device].blob = nullptr;
    g_noalloc[device].blob_bytes = 0;
    return BF_OK;
}

int bf_noalloc_status(int device, int* status) {
    if (status == nullptr) return fail(BF_EINVAL, "status is null");
    if (device < 0 || device >= kNoAllocMaxDevices) return fail(BF_EINVAL, "device index out of range");
    BF_ON_DEVICE(device);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        NoAllocDevice* d = nullptr;
        const int rc = noalloc_setup(device, &d);
        if (rc != BF_OK) return rc;
        scratch = d->scratch;
    }
    BF_CUDA(cudaDeviceSynchronize());
    BF_CUDA(cudaMemcpy(status, scratch, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status != 0) {
        BF_CUDA(cudaMemset(scratch, 0, sizeof(int)));
        return fail(BF_EDEVICE, "a device-side bounded wait ran out (code " + std::to_string(*status) + ")");
    }
    return BF_OK;
}

}  // extern "C"
