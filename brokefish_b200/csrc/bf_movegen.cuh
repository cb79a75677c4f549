// Legal-move generation for the 32-slot piece-list board, one warp per board, lane = slot.
//
// The contract of the reference's engine (brokefish/env/torch_impl.py:254-291, csrc/movegen.cuh):
// `mask [n,32]` 64-bit words, bit s of word p set when the piece in slot p may legally move to
// square s, and `in_check [n]` for the side to move.  A promotion is one bit (the type travels
// beside the move); castling is the king's two-square move; en passant is a pawn's diagonal move
// onto an empty square.
//
// Piece word (brokefish/env/torch_impl.py:40-47): bits 0-5 square (rank * 8 + file), 6-8 type
// (0 pawn, 1 knight, 2 bishop, 3 rook, 4 queen, 5 king), bit 9 "special" (king, rook: has moved;
// pawn: has just made its double step), bit 10 colour (1 black), bit 11 captured.  The control
// word's sign is the side to move (negative: black).
//
// Method: pseudo-legal targets from bitboards built with warp-wide OR reductions, then every
// candidate is tested by removing / adding the squares it changes and asking whether the
// mover's king square is attacked (rays from the king outwards, knight / king / pawn patterns),
// which decides exactly what the reference decides by replaying each move and building the
// opponent's control map (torch_impl.py:266-290).  Castling tests the king's start, crossed and
// landing squares in the position after the move, as the reference does.
#pragma once
#include <stdint.h>

namespace bfmg {

constexpr unsigned long long kFileA = 0x0101010101010101ull, kFileH = kFileA << 7;
constexpr unsigned kFull = 0xffffffffu;
enum { PAWN = 0, KNIGHT = 1, BISHOP = 2, ROOK = 3, QUEEN = 4, KING = 5 };

__device__ __forceinline__ unsigned long long warp_or(unsigned long long v) {
    const unsigned lo = __reduce_or_sync(kFull, static_cast<unsigned>(v));
    const unsigned hi = __reduce_or_sync(kFull, static_cast<unsigned>(v >> 32));
    return (static_cast<unsigned long long>(hi) << 32) | lo;
}
__device__ __forceinline__ unsigned long long knight_pattern(unsigned long long b) {
    const unsigned long long l1 = (b >> 1) & ~kFileH, l2 = (b >> 2) & ~(kFileH | (kFileH >> 1));
    const unsigned long long r1 = (b << 1) & ~kFileA, r2 = (b << 2) & ~(kFileA | (kFileA << 1));
    const unsigned long long h1 = l1 | r1, h2 = l2 | r2;
    return (h1 << 16) | (h1 >> 16) | (h2 << 8) | (h2 >> 8);
}
__device__ __forceinline__ unsigned long long king_pattern(unsigned long long b) {
    const unsigned long long row = b | ((b >> 1) & ~kFileH) | ((b << 1) & ~kFileA);
    return (row | (row << 8) | (row >> 8)) & ~b;
}
// Squares seen from `sq` along the rook (diag = false) or bishop (diag = true) lines, each ray
// ending on and including its first occupied square.
__device__ __forceinline__ unsigned long long rays(int sq, unsigned long long occ, bool diag) {
    const int r0 = sq >> 3, f0 = sq & 7;
    unsigned long long out = 0ull;
#pragma unroll
    for (int d = 0; d < 4; ++d) {
        const int dr = diag ? ((d & 1) ? 1 : -1) : (d == 0 ? 1 : (d == 1 ? -1 : 0));
        const int df = diag ? ((d & 2) ? 1 : -1) : (d == 2 ? 1 : (d == 3 ? -1 : 0));
        int r = r0 + dr, f = f0 + df;
        while (r >= 0 && r < 8 && f >= 0 && f < 8) {
            const unsigned long long bit = 1ull << (r * 8 + f);
            out |= bit;
            if (occ & bit) break;
            r += dr; f += df;
        }
    }
    return out;
}

// The opponent's pieces by the way they attack.
struct Enemy {
    unsigned long long pawns, knights, diag, line, king;
    bool black;                 // the opponent's colour
};

__device__ __forceinline__ bool attacked(int sq, unsigned long long occ, const Enemy& e) {
    const unsigned long long b = 1ull << sq;
    if (knight_pattern(b) & e.knights) return true;
    if (king_pattern(b) & e.king) return true;
    // a black pawn stands one rank above the square it attacks, a white pawn one rank below
    const unsigned long long from = e.black ? (((b << 7) & ~kFileH) | ((b << 9) & ~kFileA))
                                            : (((b >> 7) & ~kFileA) | ((b >> 9) & ~kFileH));
    if (from & e.pawns) return true;
    if (rays(sq, occ, false) & e.line) return true;
    return (rays(sq, occ, true) & e.diag) != 0ull;
}
__device__ __forceinline__ Enemy without(const Enemy& e, unsigned long long gone) {
    Enemy r = e;
    r.pawns &= ~gone; r.knights &= ~gone; r.diag &= ~gone; r.line &= ~gone; r.king &= ~gone;
    return r;
}

// Warp-collective: every lane passes its slot's piece word; returns this slot's legal-target
// word.  `in_check` (same value on every lane) says whether the side to move is in check.
__device__ __forceinline__ unsigned long long legal_word(unsigned word, int control, bool& in_check) {
    const bool black = control < 0;
    const bool live = ((word >> 11) & 1u) == 0u;
    const bool is_black = (word >> 10) & 1u;
    const bool special = (word >> 9) & 1u;
    const int type = (word >> 6) & 7;
    const int sq = word & 63;
    const bool mine = live && (is_black == black);
    const bool theirs = live && (is_black != black);
    const unsigned long long bb = live ? (1ull << sq) : 0ull;

    const unsigned long long occ = warp_or(bb);
    const unsigned long long own = warp_or(mine ? bb : 0ull);
    const unsigned long long opp = occ & ~own;
    Enemy e;
    e.black = !black;
    e.pawns = warp_or(theirs && type == PAWN ? bb : 0ull);
    e.knights = warp_or(theirs && type == KNIGHT ? bb : 0ull);
    e.diag = warp_or(theirs && (type == BISHOP || type == QUEEN) ? bb : 0ull);
    e.line = warp_or(theirs && (type == ROOK || type == QUEEN) ? bb : 0ull);
    e.king = warp_or(theirs && type == KING ? bb : 0ull);
    const unsigned long long ep_pawns = warp_or(theirs && type == PAWN && special ? bb : 0ull);
    const unsigned long long fresh_rooks = warp_or(mine && type == ROOK && !special ? bb : 0ull);
    const unsigned long long my_king = warp_or(mine && type == KING ? bb : 0ull);
    const int king_sq = my_king ? __ffsll(static_cast<long long>(my_king)) - 1 : 0;
    in_check = my_king != 0ull && attacked(king_sq, occ, e);
    if (!mine) return 0ull;

    // ---- pseudo-legal targets ----
    const int rank = sq >> 3, file = sq & 7;
    unsigned long long cand = 0ull, ep_target = 0ull;
    if (type == KNIGHT) {
        cand = knight_pattern(bb);
    } else if (type == KING) {
        cand = king_pattern(bb);
        if (!special) {
            const int row = black ? 56 : 0;
            if ((fresh_rooks >> (row + 7)) & 1ull)
                if (((occ >> (row + 5)) & 3ull) == 0ull) cand |= 1ull << (row + 6);
            if ((fresh_rooks >> row) & 1ull)
                if (((occ >> (row + 1)) & 7ull) == 0ull) cand |= 1ull << (row + 2);
        }
    } else if (type == PAWN) {
        const int up = black ? -8 : 8;
        const int f1 = sq + up;
        if (f1 >= 0 && f1 < 64 && !((occ >> f1) & 1ull)) {
            cand |= 1ull << f1;
            const bool start = black ? rank == 6 : rank == 1;
            if (start && !((occ >> (f1 + up)) & 1ull)) cand |= 1ull << (f1 + up);
        }
        if (f1 >= 0 && f1 < 64) {
            if (file > 0) cand |= (1ull << (f1 - 1)) & opp;
            if (file < 7) cand |= (1ull << (f1 + 1)) & opp;
            // en passant: an enemy pawn that has just made its double step stands beside us
            if (rank == (black ? 3 : 4)) {
                if (file > 0 && ((ep_pawns >> (sq - 1)) & 1ull)) ep_target |= 1ull << (f1 - 1);
                if (file < 7 && ((ep_pawns >> (sq + 1)) & 1ull)) ep_target |= 1ull << (f1 + 1);
                cand |= ep_target;
            }
        }
    } else {
        if (type == BISHOP || type == QUEEN) cand |= rays(sq, occ, true);
        if (type == ROOK || type == QUEEN) cand |= rays(sq, occ, false);
    }
    cand &= ~own;

    // ---- king safety, candidate by candidate ----
    unsigned long long legal = 0ull;
    for (unsigned long long rest = cand; rest != 0ull; rest &= rest - 1ull) {
        const int t = __ffsll(static_cast<long long>(rest)) - 1;
        const unsigned long long tb = 1ull << t;
        bool ok;
        if (type == KING && (t - sq == 2 || sq - t == 2)) {
            // castling: the rook jumps over the king; the king's start, crossed and landing
            // squares must not be attacked in the position after the move
            const int row = sq & 56;
            const bool kingside = t > sq;
            const unsigned long long rook_from = 1ull << (kingside ? row + 7 : row);
            const unsigned long long rook_to = 1ull << (kingside ? row + 5 : row + 3);
            const unsigned long long after = (occ & ~bb & ~rook_from) | tb | rook_to;
            const int lo = kingside ? sq : t;
            ok = !attacked(lo, after, e) && !attacked(lo + 1, after, e) && !attacked(lo + 2, after, e);
        } else {
            unsigned long long gone = tb & opp;
            if (type == PAWN && (ep_target & tb)) gone = 1ull << (t - (black ? -8 : 8));
            const unsigned long long after = ((occ & ~bb) & ~gone) | tb;
            ok = my_king == 0ull || !attacked(type == KING ? t : king_sq, after, without(e, gone));
        }
        if (ok) legal |= tb;
    }
    return legal;
}

// One warp per board.
__global__ void __launch_bounds__(128) movegen_kernel(const uint16_t* __restrict__ boards,
                                                      const int16_t* __restrict__ control, int n,
                                                      unsigned long long* __restrict__ mask,
                                                      unsigned char* __restrict__ in_check) {
    const int board = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (board >= n) return;
    bool chk;
    const unsigned long long w = legal_word(boards[static_cast<size_t>(board) * 32 + lane], control[board], chk);
    mask[static_cast<size_t>(board) * 32 + lane] = w;
    if (in_check != nullptr && lane == 0) in_check[board] = chk ? 1 : 0;
}

}  // namespace bfmg
