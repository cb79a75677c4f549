// Row-warp code of the small-batch form of the int8 evaluator: ONE board per tile (included by
// bf_encoder.cu).
//
// A tile's latency is the length of one row warp's instruction chain through the layers, whatever
// is in the tile, so a batch that leaves SMs idle (at most one board per SM) is better served by
// sixteen warps per BOARD than by four.  The MMA still wants 128 rows, so the board's 32 rows are
// written four times into the A operand (rows lane, 32 + lane, 64 + lane, 96 + lane) and every lane
// quadrant of tensor memory receives a full copy of every GEMM's output.  Warp (q, qt) then works
// on board row `lane` through quadrant q and owns ONE 16-column piece of every 256-wide row:
// columns 128 (q >> 1) + 32 qt + 16 (q & 1) .. +15 -- the sixteen pieces the four quarter-threads
// of a row own in the four-board kernel, dealt out to sixteen threads.  Its residual-stream piece
// lives in its own quadrant's columns; what another quadrant holds there is never read.  Weight
// stream, MMA issue and tensor-memory map are those of the four-board kernel; the arithmetic is
// the same, bit for bit.
//
// Exchanges are sixteen-way, across the CTA's row warps (named barrier 5, 512 threads).  Attention
// is split by head pair: quadrant j drains QKV unit j from its own copy of the accumulator and runs
// pair j's four attention units on its own rows of the staging blocks with the four-board kernel's
// own code, the four pairs side by side; the head epilogue runs on quadrant 0's four warps.
#pragma once

namespace bf {
namespace one {

// the 16 KB exchange region: row maxima [2 parity][16 threads][32 rows] floats (4 KB), then the
// norm's partial sums and sums of squares [32 summation lanes][32 rows] floats (4 KB each) and
// its (min, max) pairs [16 threads][32 rows] x 8 B (4 KB)
constexpr uint32_t X_MAX = 0, X_SUM = 4096, X_SQ = 8192, X_MM = 12288;

__device__ __forceinline__ void rows_sync() { named_bar_sync(5, 512); }
__device__ __forceinline__ int thread16(const RowCtx& c) { return 4 * c.q + c.qt; }
// first column of this thread's piece of a 256-wide row
__device__ __forceinline__ int piece_col(const RowCtx& c) { return 128 * (c.q >> 1) + 32 * c.qt + 16 * (c.q & 1); }

__device__ __forceinline__ float exchange_max16(RowCtx& c, float mine) {
    const uint32_t base = c.smem + SM_XCH + X_MAX + 4u * (c.xpar * 512 + c.lane);
    sts32(base + 128u * thread16(c), __float_as_uint(mine));
    rows_sync();
    float m = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        uint32_t v;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(base + 128u * k) : "memory");
        m = fmaxf(m, __uint_as_float(v));
    }
    c.xpar ^= 1;
    return m;
}

// 16 quantised bytes into the four row copies of an A-operand K-slab
__device__ __forceinline__ void store_copies(uint32_t slab, int lane, int chunk, uint4 v) {
#pragma unroll
    for (int k = 0; k < 4; ++k) sts128(slab + sw_off(32 * k + lane, chunk), v);
}
// An accumulator slot this warp does not read is handed back at once (the barrier counts all
// sixteen row warps).
__device__ __forceinline__ void skip_slot(RowCtx& c, int slot) {
    if (slot) ++c.full1; else ++c.full0;
    __syncwarp();
    if (c.lane == 0) mbar_arrive(bar_addr(c.smem, B_ACC_EMPTY + slot));
}

// One LayerNorm for this thread's 16 columns; summation order and arithmetic as `ln_stage`.  The
// thread's columns are the reference's summation lanes l0 = 16 u + 4 qt + 2 half and l0 + 1; it
// publishes their partial sums, every thread of the row then combines all 32 by the butterfly
// 16, 8, 4, 2, 1.
template <bool kFinal>
__device__ __forceinline__ float ln_stage(RowCtx& c, const Params& p) {
    const int col = piece_col(c), l0 = col >> 3;
    uint32_t x[8];
    tmem_ld8(c.tm + TM_X + (col >> 1), x);
    tmem_wait_ld();
    const uint32_t xch = c.smem + SM_XCH;
    {
        // lanes (l0, l0 + 1) ride in one packed register: words 0-3 are lane l0's eight columns
        uint64_t s2 = pk2(0.f, 0.f), q2 = pk2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            uint64_t f = h2_to_f2(__byte_perm(x[k], x[4 + k], 0x5410));
            s2 = add2(s2, f);
            q2 = fma2(f, f, q2);
            f = h2_to_f2(__byte_perm(x[k], x[4 + k], 0x7632));
            s2 = add2(s2, f);
            q2 = fma2(f, f, q2);
        }
        __half2 mn = as_h2(x[0]), mx = as_h2(x[0]);
#pragma unroll
        for (int i = 1; i < 8; ++i) {
            mn = __hmin2(mn, as_h2(x[i]));
            mx = __hmax2(mx, as_h2(x[i]));
        }
        float a, b;
        upk2(s2, a, b);
        sts32(xch + X_SUM + 4u * (32 * l0 + c.lane), __float_as_uint(a));
        sts32(xch + X_SUM + 4u * (32 * (l0 + 1) + c.lane), __float_as_uint(b));
        upk2(q2, a, b);
        sts32(xch + X_SQ + 4u * (32 * l0 + c.lane), __float_as_uint(a));
        sts32(xch + X_SQ + 4u * (32 * (l0 + 1) + c.lane), __float_as_uint(b));
        const uint32_t mm = xch + X_MM + 8u * (32 * thread16(c) + c.lane);
        sts32(mm, __float_as_uint(fminf(__low2float(mn), __high2float(mn))));
        sts32(mm + 4, __float_as_uint(fmaxf(__low2float(mx), __high2float(mx))));
    }
    rows_sync();
    float tot, totq, xmin, xmax;
    {
        auto ld = [&](uint32_t off) {
            uint32_t v;
            asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(off) : "memory");
            return __uint_as_float(v);
        };
        // butterfly over the 32 lane partials P[l]: level 16 pairs l with l + 16, level 8 l with
        // l + 8, ...; every level halves the set and the last add gives the total
        auto butterfly = [&](uint32_t base) {
            float v[16];
#pragma unroll
            for (int l = 0; l < 16; ++l) v[l] = __fadd_rn(ld(base + 4u * (32 * l + c.lane)), ld(base + 4u * (32 * (l + 16) + c.lane)));
#pragma unroll
            for (int l = 0; l < 8; ++l) v[l] = __fadd_rn(v[l], v[l + 8]);
#pragma unroll
            for (int l = 0; l < 4; ++l) v[l] = __fadd_rn(v[l], v[l + 4]);
            v[0] = __fadd_rn(v[0], v[2]);
            v[1] = __fadd_rn(v[1], v[3]);
            return __fadd_rn(v[0], v[1]);
        };
        tot = butterfly(xch + X_SUM);
        totq = butterfly(xch + X_SQ);
        xmin = ld(xch + X_MM + 8u * c.lane);
        xmax = ld(xch + X_MM + 8u * c.lane + 4);
#pragma unroll
        for (int k = 1; k < 16; ++k) {
            xmin = fminf(xmin, ld(xch + X_MM + 8u * (32 * k + c.lane)));
            xmax = fmaxf(xmax, ld(xch + X_MM + 8u * (32 * k + c.lane) + 4));
        }
    }
    const float mean = __fmul_rn(tot, 1.0f / 256.0f);
    const float var = fmaxf(__fsub_rn(__fmul_rn(totq, 1.0f / 256.0f), __fmul_rn(mean, mean)), 0.f);
    const float rstd = p.rsqrt_rn ? __frsqrt_rn(__fadd_rn(var, p.eps)) : rsqrtf(__fadd_rn(var, p.eps));
    const float e_lo = __half2float(__float2half_rn(__fmul_rn(__fsub_rn(xmin, mean), rstd)));
    const float e_hi = __half2float(__float2half_rn(__fmul_rn(__fsub_rn(xmax, mean), rstd)));
    const float amax = fmaxf(fabsf(e_lo), fabsf(e_hi));
    const float sc = amax > 0.f ? __fdiv_rn(amax, kQMaxS8) : 1.0f;
    const uint64_t nmean2 = pk2(-mean, -mean), rstd2 = pk2(rstd, rstd);
    if (!kFinal) {
        const float inv = __fdiv_rn(1.0f, sc);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = f2_to_h2(mul2(add2(h2_to_f2(x[i]), nmean2), rstd2));
        store_copies(c.sm_a + (col >> 7) * 16384, c.lane, (col & 127) >> 4, quant16(x, inv, c.one2));
    } else {
        const uint4* g4 = reinterpret_cast<const uint4*>(p.tail + col);
        const uint4* b4 = reinterpret_cast<const uint4*>(p.tail + kD + col);
#pragma unroll
        for (int v = 0; v < 2; ++v) {
            const uint4 gv = __ldg(g4 + v), bv = __ldg(b4 + v);
            const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                x[4 * v + j] = f2_to_h2(fma2(mul2(add2(h2_to_f2(x[4 * v + j]), nmean2), rstd2),
                                             h2_to_f2(gw[j]), h2_to_f2(bw[j])));
            // head A operand: K-slab col / 64, 16-byte group (col % 64) / 8 + v
            store_copies(c.sm_r + (col >> 6) * 16384, c.lane, ((col & 63) >> 3) + v,
                         make_uint4(x[4 * v], x[4 * v + 1], x[4 * v + 2], x[4 * v + 3]));
        }
    }
    return sc;
}

__device__ __forceinline__ void attention_block(RowCtx& c, const Params& p, const LayerParams& lp, float sa,
                                                uint32_t alive) {
    // Head pair j is quadrant j's: its four warps drain QKV unit j from their own copy of the
    // accumulator (48 of the 192 columns each, as a board's four warps do in the four-board
    // kernel), stage Q, K and V in their own 32 rows of the staging blocks and run the pair's four
    // attention units there, all four pairs side by side.  The other quadrants only account for a
    // unit: they wait for it and hand the accumulator back (the barrier counts sixteen warps, and
    // an arrival must fall into its own unit's phase).
    const int j = c.q;
#pragma unroll 1
    for (int u = 0; u < 4; ++u) {
        row_wait_acc<false>(c, 0, PH_LN);
        if (u != j) {
            row_release_acc(c, 0);
            continue;
        }
        // all 48 columns are fetched at once and the accumulator goes back before they are worked
        // on: the next unit's product runs under this one's descale
        uint32_t acc[3][16];
        tmem_ld16(c.tm + TM_ACC + 48 * c.qt, acc[0]);
        tmem_ld16(c.tm + TM_ACC + 48 * c.qt + 16, acc[1]);
        tmem_ld16(c.tm + TM_ACC + 48 * c.qt + 32, acc[2]);
        row_release_acc(c, 0);             // waits for the loads
#pragma unroll
        for (int g = 0; g < 3; ++g) {
            const int c0 = 48 * c.qt + 16 * g, m = c0 >> 6, cm = c0 & 63;
            uint32_t h[8];
            descale<16, false, kAccInt>(acc[g], sa, __ldg(lp.sw_qkv + m * 2 + (j >> 1)), lp.b_qkv + j * 192 + c0, h);
#pragma unroll
            for (int k = 0; k < 2; ++k)
                sts128(c.sm_r + m * 16384 + sw_off(c.row, (cm >> 3) + k),
                       make_uint4(h[4 * k], h[4 * k + 1], h[4 * k + 2], h[4 * k + 3]));
        }
    }
    board_sync(c);                         // this pair's Q/K/V rows are staged
    attention_unit(c, alive);
    board_sync(c);                         // the pair's outputs are in the output block
    {
        // this thread's 16 of the row's 256 attention outputs: columns 64 j + 16 qt .. +15.  The row
        // maximum goes through the sixteen-way exchange, the quantised piece into all four row
        // copies of the out-projection's A operand.
        uint32_t oh[8];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const uint4 v = lds128(c.sm_r + 49152 + sw_off(c.row, 2 * c.qt + k));
            oh[4 * k] = v.x; oh[4 * k + 1] = v.y; oh[4 * k + 2] = v.z; oh[4 * k + 3] = v.w;
        }
        const float amax = exchange_max16(c, amax_h2<8>(oh, true));
        sa = amax > 0.f ? __fdiv_rn(amax, kQMaxS8) : 1.0f;
        const float inv = __fdiv_rn(1.0f, sa);
        store_copies(c.sm_a + (j >> 1) * 16384, c.lane, 4 * (j & 1) + c.qt, quant16(oh, inv, c.one2));
        row_publish(c, B_A_READY);
    }
    // out-projection: this thread's piece of slot q >> 1
    const int u = c.q >> 1, col = piece_col(c);
    row_wait_acc<false>(c, u, PH_O_QUANT);
    {
        uint32_t acc[16], y[8], xo[8];
        tmem_ld16(c.tm + TM_ACC + col, acc);
        tmem_ld8(c.tm + TM_X + (col >> 1), xo);
        tmem_wait_ld();
        row_release_acc(c, u);
        skip_slot(c, 1 - u);
        descale<16, false, kAccInt>(acc, sa, __ldg(lp.sw_o + u), lp.b_o + col, y);
#pragma unroll
        for (int i = 0; i < 8; ++i) xo[i] = as_u32(__hadd2(as_h2(xo[i]), as_h2(y[i])));
        tmem_st8(c.tm + TM_X + (col >> 1), xo);
    }
    tmem_wait_st();
}

__device__ __forceinline__ void ffn_block(RowCtx& c, const Params& p, const LayerParams& lp, float sa) {
    float sa2_0 = 1.f, sa2_1 = 1.f;
    const int u = c.q >> 1, col = piece_col(c);
    const uint32_t t0 = c.tm + TM_ACC + col;
#pragma unroll 1
    for (int st = 0; st < 8; ++st) {
        const int kind2 = (0xD4 >> st) & 1;
        const int ch = kind2 ? ((0x32010000u >> (4 * st)) & 0xF) : ((0x00302010u >> (4 * st)) & 0xF);
        row_wait_acc<false>(c, u, PH_FF1_EPI);
        if (!kind2) {
            uint32_t acc[16], hid[8];
            tmem_ld16(t0, acc);
            tmem_wait_ld();
            row_release_acc(c, u);
            skip_slot(c, 1 - u);
            descale<16, true, kAccInt>(acc, sa, __ldg(lp.sw_ff1 + 2 * ch + u), lp.b_ff1 + 256 * ch + col, hid);
            const float amax = exchange_max16(c, amax_h2<8>(hid, false));
            const float sc = amax > 0.f ? __fdiv_rn(amax, kQMaxU8) : 1.0f;
            const float inv = __fdiv_rn(1.0f, sc);
            if (ch & 1) sa2_1 = sc; else sa2_0 = sc;
            store_copies(c.sm_r + (ch & 1) * 32768 + u * 16384, c.lane, (col & 127) >> 4, quant16(hid, inv, c.one2));
            row_publish(c, B_A2_READY + (ch & 1));
        } else {
            const float s1 = (ch & 1) ? sa2_1 : sa2_0;
            const float s2 = __ldg(lp.sw_ff2 + u);
            const uint64_t s1_2 = pk2(s1, s1), s2_2 = pk2(s2, s2);
            uint32_t acc[16], run[8];
            tmem_ld16(t0, acc);
            if (ch > 0) tmem_ld8(c.tm + TM_OY + (col >> 1), run);
            tmem_wait_ld();
            row_release_acc(c, u);
            skip_slot(c, 1 - u);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                uint64_t f = pk2(static_cast<float>(static_cast<int>(acc[2 * i])),
                                 static_cast<float>(static_cast<int>(acc[2 * i + 1])));
                f = mul2(f, s1_2);
                f = ch > 0 ? fma2(f, s2_2, h2_to_f2(run[i])) : mul2(f, s2_2);
                run[i] = f2_to_h2(f);
            }
            if (ch < 3) {
                tmem_st8(c.tm + TM_OY + (col >> 1), run);
            } else {
                uint32_t xo[8];
                tmem_ld8(c.tm + TM_X + (col >> 1), xo);
                tmem_wait_ld();
                const uint4* b4 = reinterpret_cast<const uint4*>(lp.b_ff2 + col);
#pragma unroll
                for (int v = 0; v < 2; ++v) {
                    const uint4 bv = __ldg(b4 + v);
                    const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int i = 4 * v + k;
                        xo[i] = as_u32(__hadd2(as_h2(xo[i]), __hadd2(as_h2(run[i]), as_h2(bw[k]))));
                    }
                }
                tmem_st8(c.tm + TM_X + (col >> 1), xo);
            }
            tmem_wait_st();
        }
    }
}

// One tile = one board.  `head` is the four-board kernel's head epilogue, run by quadrant 0.
template <class HeadFn>
__device__ __forceinline__ void row_warps_tile(RowCtx& c, const Params& p, int tile, HeadFn&& head) {
    c.valid = tile < c.n;
    const int board = (c.valid && p.leaf_index != nullptr) ? __ldg(p.leaf_index + tile) : tile;
    c.grow = static_cast<long>(board) * kT + c.lane;
    const uint32_t word = c.valid ? p.boards[c.grow] : 0u;
    const uint32_t alive = __ballot_sync(0xffffffffu, ((word >> 11) & 1u) == 0u);
    const int ctl = c.valid ? static_cast<int>(p.control[board]) : 1;
    const int col = piece_col(c);
    {
        const int stm = ctl < 0;
        const int clk = min(max((ctl < 0 ? -ctl : ctl) - 1, 0), kNClock - 1);
        const int rp = min(c.valid ? static_cast<int>(p.rep[board]) : 0, kNRep - 1);
        c.word = word; c.stm = stm; c.clk = clk; c.rp = rp;
        const int sq = word & 63;
        const int ts = min(static_cast<int>(((word >> 6) & 7) * 2 + ((word >> 9) & 1)), kNTypeSpecial - 1);
        const int ct = ((word >> 10) & 1) * 2 + stm;
        const uint4* e_sq = reinterpret_cast<const uint4*>(p.emb + (EMB_SQUARE + sq) * kD + col);
        const uint4* e_ts = reinterpret_cast<const uint4*>(p.emb + (EMB_TS + ts) * kD + col);
        const uint4* e_ct = reinterpret_cast<const uint4*>(p.emb + (EMB_CT + ct) * kD + col);
        const uint4* e_ck = reinterpret_cast<const uint4*>(p.emb + (EMB_CLOCK + clk) * kD + col);
        const uint4* e_rp = reinterpret_cast<const uint4*>(p.emb + (EMB_REP + rp) * kD + col);
        uint32_t e8[8];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
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
                e8[4 * k + j] = as_u32(x);
            }
        }
        tmem_st8(c.tm + TM_X + (col >> 1), e8);
        tmem_wait_st();
    }
#pragma unroll 1
    for (int layer = 0; layer < p.n_layers; ++layer) {
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
        float sa = ln_stage<false>(c, p);
        row_publish(c, B_A_READY);
        attention_block(c, p, lp, sa, c.valid ? alive : 0xffffffffu);
        sa = ln_stage<false>(c, p);
        row_publish(c, B_A_READY);
        ffn_block(c, p, lp, sa);
    }
    ln_stage<true>(c, p);
    row_publish(c, B_A_READY);                           // the head product's A operand
    if (c.q == 0) {
        head(c, board, word, ctl, alive);
    } else {
        // the other quadrants only account for the head product and hand its accumulator back
        row_wait_acc<false>(c, 0, PH_LN);
        row_release_acc(c, 0);
    }
}

}  // namespace one
}  // namespace bf
