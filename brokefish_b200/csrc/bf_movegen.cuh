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
// Method: bitboards built with warp-wide OR reductions; every enemy lane contributes the squares
// its piece attacks with the mover's king lifted off the board (king moves and castling avoid
// their union); the enemy lanes that attack the king are the checkers (one checker: the other
// pieces may only capture it or step between; two: only the king moves); every lane walks the
// line from the king to its own piece, which finds the pieces that shield the king from a slider
// (they move only along that line) and, for a checking slider, the squares between.  Only en
// passant, which takes two pieces off one rank at once, is tested on the position after the
// move.  This decides what the reference decides by replaying each move and building the
// opponent's control map (torch_impl.py:266-290).
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
    const int rank = sq >> 3, file = sq & 7;

    // ---- what the opponent attacks, with the mover's king lifted off the board (so that a
    //      square behind the king on a checking line counts as attacked) ----
    unsigned long long att = 0ull;
    if (theirs) {
        const unsigned long long occ_nk = occ & ~my_king;
        if (type == PAWN)
            att = is_black ? (((bb >> 9) & ~kFileH) | ((bb >> 7) & ~kFileA))
                           : (((bb << 7) & ~kFileH) | ((bb << 9) & ~kFileA));
        else if (type == KNIGHT) att = knight_pattern(bb);
        else if (type == KING) att = king_pattern(bb);
        else {
            if (type == BISHOP || type == QUEEN) att |= rays(sq, occ_nk, true);
            if (type == ROOK || type == QUEEN) att |= rays(sq, occ_nk, false);
        }
    }
    const unsigned long long danger = warp_or(att);
    in_check = (danger & my_king) != 0ull;
    const unsigned checkers = __ballot_sync(kFull, theirs && (att & my_king) != 0ull);

    // ---- the line from the king to this piece, when the piece is the first one met on a rank,
    //      file or diagonal through the king: `line_to_me` = squares after the king up to and
    //      including the piece, `beyond` = the next piece on the same ray, `line` = everything
    //      walked, from the king's neighbour to that next piece ----
    unsigned long long line = 0ull, line_to_me = 0ull, beyond = 0ull;
    bool first_on_ray = false, ray_diag = false;
    if (live && my_king != 0ull && bb != my_king) {
        const int kr = king_sq >> 3, kf = king_sq & 7;
        const int dr = rank - kr, df = file - kf;
        const bool aligned = (dr == 0) != (df == 0) || (dr != 0 && (dr == df || dr == -df));
        if (aligned) {
            const int sr = (dr > 0) - (dr < 0), sf = (df > 0) - (df < 0);
            ray_diag = sr != 0 && sf != 0;
            int r = kr + sr, f = kf + sf;
            bool past = false;
            while (r >= 0 && r < 8 && f >= 0 && f < 8) {
                const unsigned long long bit = 1ull << (r * 8 + f);
                line |= bit;
                if (!past) line_to_me |= bit;
                if (occ & bit) {
                    if (!past) {
                        if (bit != bb) break;          // something stands between the king and this piece
                        past = first_on_ray = true;
                    } else {
                        beyond = bit;
                        break;
                    }
                }
                r += sr; f += sf;
            }
        }
    }
    // one checker: the other pieces may only capture it or step between it and the king
    unsigned long long target_mask = ~0ull;
    const int n_checkers = __popc(checkers);
    {
        const bool slider = type == BISHOP || type == ROOK || type == QUEEN;
        const unsigned long long blk = (slider && first_on_ray) ? line_to_me : bb;
        const int c = checkers ? __ffs(checkers) - 1 : 0;
        const unsigned lo = __shfl_sync(kFull, static_cast<unsigned>(blk), c);
        const unsigned hi = __shfl_sync(kFull, static_cast<unsigned>(blk >> 32), c);
        if (n_checkers == 1) target_mask = (static_cast<unsigned long long>(hi) << 32) | lo;
        else if (n_checkers > 1) target_mask = 0ull;
    }
    if (!mine) return 0ull;

    // ---- pseudo-legal targets ----
    unsigned long long cand = 0ull, ep_target = 0ull;
    if (type == KNIGHT) {
        cand = knight_pattern(bb);
    } else if (type == KING) {
        cand = king_pattern(bb) & ~danger;
        // castling: neither the king's square nor the one it crosses nor the one it lands on may
        // be attacked (on the first rank nothing the rook's jump uncovers or covers changes that)
        if (!special && !in_check) {
            const int row = black ? 56 : 0;
            if ((fresh_rooks >> (row + 7)) & 1ull)
                if (((occ >> (row + 5)) & 3ull) == 0ull && ((danger >> (row + 5)) & 3ull) == 0ull)
                    cand |= 1ull << (row + 6);
            if ((fresh_rooks >> row) & 1ull)
                if (((occ >> (row + 1)) & 7ull) == 0ull && ((danger >> (row + 2)) & 3ull) == 0ull)
                    cand |= 1ull << (row + 2);
        }
        return cand & ~own;
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
            }
        }
    } else {
        if (type == BISHOP || type == QUEEN) cand |= rays(sq, occ, true);
        if (type == ROOK || type == QUEEN) cand |= rays(sq, occ, false);
    }
    cand &= ~own;
    if (my_king == 0ull) return cand | (ep_target & ~own);  // no king to protect
    // a piece that shields the king from a slider moves only along the shielding line
    const bool pinned = first_on_ray && (beyond & (ray_diag ? e.diag : e.line)) != 0ull;
    unsigned long long legal = cand & target_mask & (pinned ? line : ~0ull);
    // en passant takes two pieces off one rank at once: tested on the position after the move
    for (unsigned long long rest = ep_target & ~own; rest != 0ull; rest &= rest - 1ull) {
        const int t = __ffsll(static_cast<long long>(rest)) - 1;
        const unsigned long long tb = 1ull << t;
        const unsigned long long gone = 1ull << (t - (black ? -8 : 8));
        const unsigned long long after = ((occ & ~bb) & ~gone) | tb;
        if (!attacked(king_sq, after, without(e, gone))) legal |= tb;
    }
    return legal;
}

// Castling rights of a board in FEN order KQkq as four bits (torch_impl.py:294-318): the king
// and that corner's rook are alive and have never moved.  Warp-collective.
__device__ __forceinline__ unsigned castling_bits(unsigned word) {
    const bool intact = ((word >> 11) & 1u) == 0u && ((word >> 9) & 1u) == 0u;
    const bool is_black = (word >> 10) & 1u;
    const int type = (word >> 6) & 7, sq = word & 63;
    const unsigned wk = __ballot_sync(kFull, intact && type == KING && !is_black) != 0u;
    const unsigned bk = __ballot_sync(kFull, intact && type == KING && is_black) != 0u;
    const bool rook = intact && type == ROOK;
    const unsigned k = __ballot_sync(kFull, rook && !is_black && sq == 7) != 0u;
    const unsigned q = __ballot_sync(kFull, rook && !is_black && sq == 0) != 0u;
    const unsigned k2 = __ballot_sync(kFull, rook && is_black && sq == 63) != 0u;
    const unsigned q2 = __ballot_sync(kFull, rook && is_black && sq == 56) != 0u;
    return (wk & k) | ((wk & q) << 1) | ((bk & k2) << 2) | ((bk & q2) << 3);
}

// Apply one move (`move` = slot * 64 + target, -1 = no move; `promo` 0..3 = N B R Q, negative =
// queen) to a board, lane = slot: the reference's `step` without its hash
// (brokefish/env/torch_impl.py:412-548).  Returns this slot's new word; `new_control` and
// `irreversible` (capture, pawn move or a change of castling rights) are the same on every lane.
__device__ __forceinline__ unsigned step_word(unsigned word, int control, int move, int promo, int lane,
                                              int& new_control, bool& irreversible) {
    new_control = control;
    irreversible = false;
    if (move < 0) return word;
    const int source = move >> 6, target = move & 63;
    const bool white = control > 0;
    const unsigned mover = __shfl_sync(kFull, word, source);
    const int mtype = (mover >> 6) & 7, from = mover & 63;
    const bool is_pawn = mtype == PAWN;
    const unsigned rights_before = castling_bits(word);
    // capture: a live piece on the target square, or for a pawn the en passant victim, which
    // carries the double-step flag and stands beside the target's file neighbour, not on it
    const bool live = ((word >> 11) & 1u) == 0u;
    const unsigned victim_word = ((white ? 3u : 1u) << 9) + static_cast<unsigned>(target + (white ? -8 : 8));
    const bool hit = (live && static_cast<int>(word & 63u) == target) || (is_pawn && word == victim_word);
    const unsigned hits = __ballot_sync(kFull, hit);
    const bool has_capture = hits != 0u;
    unsigned w = word;
    if (has_capture && lane == __ffs(hits) - 1) w = 1u << 11;
    // castling: the rook on the king's side corner jumps over (found before any square changes)
    const int dx = target - from;
    const bool castling = mtype == KING && (dx == 2 || dx == -2);
    const int corner = (white ? 0 : 56) + (dx > 0 ? 7 : 0);
    const unsigned rooks = __ballot_sync(kFull, ((w >> 6) & 7u) == ROOK && static_cast<int>(word & 63u) == corner);
    if (lane == source) {
        w = (w & ~63u & 0xFFFu) + static_cast<unsigned>(target);
        if (is_pawn && (target >> 3) == (white ? 7 : 0))
            w += static_cast<unsigned>(promo < 0 ? QUEEN : promo + KNIGHT) << 6;
        if (mtype == KING || mtype == ROOK) w |= 1u << 9;
    }
    if (castling && rooks != 0u && lane == __ffs(rooks) - 1)
        w = (w & ~63u & 0xFFFu) + static_cast<unsigned>((white ? 0 : 56) + (dx > 0 ? 5 : 3));
    // the en passant flag lives for one ply: clear every pawn's, set the double-stepper's
    if (((w >> 6) & 7u) == PAWN) w &= ~(1u << 9) & 0xFFFu;
    if (lane == source && is_pawn && (dx == 16 || dx == -16)) w |= 1u << 9;
    const int mag = (has_capture || is_pawn) ? 1 : (control < 0 ? -control : control) + 1;
    new_control = white ? -mag : mag;
    irreversible = has_capture || is_pawn || castling_bits(w) != rights_before;
    return w;
}

// One warp per board: play `move` (with `promo`), then generate the legal moves of the result.
__global__ void __launch_bounds__(128) step_kernel(const uint16_t* __restrict__ boards,
                                                   const int16_t* __restrict__ control,
                                                   const int* __restrict__ move, const signed char* __restrict__ promo,
                                                   int n, uint16_t* __restrict__ boards_out,
                                                   int16_t* __restrict__ control_out,
                                                   unsigned char* __restrict__ irreversible,
                                                   unsigned long long* __restrict__ mask,
                                                   unsigned char* __restrict__ in_check) {
    const int board = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (board >= n) return;
    int nc;
    bool irr;
    const unsigned w = step_word(boards[static_cast<size_t>(board) * 32 + lane], control[board], move[board],
                                 promo != nullptr ? promo[board] : -1, lane, nc, irr);
    boards_out[static_cast<size_t>(board) * 32 + lane] = static_cast<uint16_t>(w);
    if (lane == 0) {
        control_out[board] = static_cast<int16_t>(nc);
        if (irreversible != nullptr) irreversible[board] = irr ? 1 : 0;
    }
    if (mask != nullptr) {
        bool chk;
        const unsigned long long m = legal_word(w, nc, chk);
        mask[static_cast<size_t>(board) * 32 + lane] = m;
        if (in_check != nullptr && lane == 0) in_check[board] = chk ? 1 : 0;
    }
}

// One warp per board: one ply of a uniform-random playout, in place.  The move is the
// floor(r * count)-th legal move in (slot, square) order (r in [0,1), product in fp32), the board
// is stepped and its new legal moves replace `mask`; a board without legal moves stays as it is
// and reports move -1.
__global__ void __launch_bounds__(128) random_ply_kernel(uint16_t* __restrict__ boards, int16_t* __restrict__ control,
                                                         unsigned long long* __restrict__ mask,
                                                         const float* __restrict__ r,
                                                         const signed char* __restrict__ promo, int n,
                                                         int* __restrict__ move_out) {
    const int board = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (board >= n) return;
    unsigned long long m = mask[static_cast<size_t>(board) * 32 + lane];
    const int cnt = __popcll(m);
    int incl = cnt;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(kFull, incl, d);
        if (lane >= d) incl += v;
    }
    const int total = __shfl_sync(kFull, incl, 31);
    int move = -1;
    if (total > 0) {
        int pick = static_cast<int>(__fmul_rn(r[board], static_cast<float>(total)));
        pick = pick < total - 1 ? pick : total - 1;
        const int k = pick - (incl - cnt);
        const unsigned owners = __ballot_sync(kFull, k >= 0 && k < cnt);
        const int owner = __ffs(owners) - 1;
        int bit = 0;
        if (lane == owner) {
            for (int i = 0; i < k; ++i) m &= m - 1ull;
            bit = __ffsll(static_cast<long long>(m)) - 1;
        }
        move = owner * 64 + __shfl_sync(kFull, bit, owner);
    }
    if (move_out != nullptr && lane == 0) move_out[board] = move;
    if (move < 0) return;
    int nc;
    bool irr, chk;
    const unsigned w = step_word(boards[static_cast<size_t>(board) * 32 + lane], control[board], move,
                                 promo != nullptr ? promo[board] : -1, lane, nc, irr);
    boards[static_cast<size_t>(board) * 32 + lane] = static_cast<uint16_t>(w);
    if (lane == 0) control[board] = static_cast<int16_t>(nc);
    mask[static_cast<size_t>(board) * 32 + lane] = legal_word(w, nc, chk);
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
