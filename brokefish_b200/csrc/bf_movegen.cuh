// Legal-move generation and move application for the 32-slot piece-list board, in two forms:
// `legal_word`, one warp per board with lane = slot (what the evaluator's expansion warp calls),
// and the stand-alone kernels further down, one thread per board.
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
// Method of the warp form: bitboards built with warp-wide OR reductions; every enemy lane contributes the squares
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

// ------------------------------------------------------------------------------------------
// One THREAD per board: the stand-alone generator.  A board is 64 bytes; with a warp per board
// every bitboard costs warp-wide reductions over 32 lanes that hold one piece each, and the
// kernel is bound by instruction issue far below the memory roof.  A thread that keeps the whole
// board needs no reductions at all: attacks of all the opponent's sliders come out of eight
// loop-free fills over the set of them at once, checkers and shielding pieces out of the same
// fills started at the king, and only the mover's own pieces are visited one by one.  Slot p has
// the same piece type on almost every board (promotions aside), so the threads of a warp take
// the same branch as they walk the slots.  Boards come in and legal words go out through shared
// memory so that global accesses stay coalesced.
// ------------------------------------------------------------------------------------------
template <int kShift>
__device__ __forceinline__ unsigned long long fill_ray(unsigned long long gen, unsigned long long occ,
                                                       unsigned long long wrap) {
    // the pieces' bits spread over empty squares in doubling steps (1, 2, 4), then one more
    // step lands on the first occupied square; `wrap` clears the file a step must not arrive on
    unsigned long long pro = ~occ & wrap;
    if constexpr (kShift > 0) {
        gen |= pro & (gen << kShift);
        pro &= pro << kShift;
        gen |= pro & (gen << (2 * kShift));
        pro &= pro << (2 * kShift);
        gen |= pro & (gen << (4 * kShift));
        return (gen << kShift) & wrap;
    } else {
        gen |= pro & (gen >> -kShift);
        pro &= pro >> -kShift;
        gen |= pro & (gen >> (-2 * kShift));
        pro &= pro >> (-2 * kShift);
        gen |= pro & (gen >> (-4 * kShift));
        return (gen >> -kShift) & wrap;
    }
}
// Squares seen from every piece of the set `b` along the bishop or the rook lines.
__device__ __forceinline__ unsigned long long fill_diag(unsigned long long b, unsigned long long occ) {
    return fill_ray<9>(b, occ, ~kFileA) | fill_ray<7>(b, occ, ~kFileH) | fill_ray<-7>(b, occ, ~kFileA) |
           fill_ray<-9>(b, occ, ~kFileH);
}
__device__ __forceinline__ unsigned long long fill_line(unsigned long long b, unsigned long long occ) {
    return fill_ray<8>(b, occ, ~0ull) | fill_ray<-8>(b, occ, ~0ull) | fill_ray<1>(b, occ, ~kFileA) |
           fill_ray<-1>(b, occ, ~kFileH);
}
// Squares a set of pawns of one colour attacks.
__device__ __forceinline__ unsigned long long pawn_attacks(unsigned long long b, bool black_pawns) {
    return black_pawns ? (((b >> 9) & ~kFileH) | ((b >> 7) & ~kFileA)) : (((b << 7) & ~kFileH) | ((b << 9) & ~kFileA));
}
// The whole rank, file or diagonal through two aligned squares (0 when they are not aligned).
__device__ __forceinline__ unsigned long long line_through(int a, int b) {
    const int ra = a >> 3, fa = a & 7, rb = b >> 3, fb = b & 7;
    if (ra == rb) return 0xFFull << (8 * ra);
    if (fa == fb) return kFileA << fa;
    if (ra - fa == rb - fb) {
        const int d = ra - fa;                                   // the a1-h8 diagonal moved up or down
        return d >= 0 ? 0x8040201008040201ull << (8 * d) : 0x8040201008040201ull >> (-8 * d);
    }
    if (ra + fa == rb + fb) {
        const int d = ra + fa - 7;                               // the h1-a8 diagonal moved up or down
        return d >= 0 ? 0x0102040810204080ull << (8 * d) : 0x0102040810204080ull >> (-8 * d);
    }
    return 0ull;
}

// One sliding piece along one line without loops or fills: on the line's squares other than the
// piece's own, subtracting the piece's bit from the occupancy flips exactly the squares up to and
// including the first occupied one above it; the same on the bit-reversed board gives the squares
// below it.
__device__ __forceinline__ unsigned long long line_attacks(unsigned long long s, unsigned long long occ,
                                                           unsigned long long line_ex) {
    const unsigned long long o = occ & line_ex;
    const unsigned long long up = o - s;
    const unsigned long long down = __brevll(__brevll(o) - __brevll(s));
    return (up ^ down) & line_ex;
}
// The rank, file and two diagonals through a square, without the square itself.
__device__ __forceinline__ unsigned long long rank_ex(int sq) { return (0xFFull << (sq & 56)) ^ (1ull << sq); }
__device__ __forceinline__ unsigned long long file_ex(int sq) { return (kFileA << (sq & 7)) ^ (1ull << sq); }
__device__ __forceinline__ unsigned long long diag_ex(int sq) {
    const int d = (sq >> 3) - (sq & 7);
    return (d >= 0 ? 0x8040201008040201ull << (8 * d) : 0x8040201008040201ull >> (-8 * d)) ^ (1ull << sq);
}
__device__ __forceinline__ unsigned long long anti_ex(int sq) {
    const int d = (sq >> 3) + (sq & 7) - 7;
    return (d >= 0 ? 0x0102040810204080ull << (8 * d) : 0x0102040810204080ull >> (-8 * d)) ^ (1ull << sq);
}

// Squares one piece `b` (a single bit) sees along the bishop or the rook lines.
__device__ __forceinline__ unsigned long long piece_diag(unsigned long long b, unsigned long long occ) {
    const int sq = __ffsll(static_cast<long long>(b)) - 1;
    return line_attacks(b, occ, diag_ex(sq)) | line_attacks(b, occ, anti_ex(sq));
}
__device__ __forceinline__ unsigned long long piece_line(unsigned long long b, unsigned long long occ) {
    const int sq = __ffsll(static_cast<long long>(b)) - 1;
    return line_attacks(b, occ, rank_ex(sq)) | line_attacks(b, occ, file_ex(sq));
}

constexpr int kTpbThreads = 128;
constexpr int kTpbInStride = 17;      // 32-bit words per board in shared memory (16 + 1: no bank conflicts)
constexpr int kTpbOutStride = 33;     // 64-bit words per board in shared memory (32 + 1)
constexpr int kTpbSmem = kTpbThreads * (kTpbInStride * 4 + kTpbOutStride * 8);

// The legal words of one board held by one thread: `my` = the board's 32 piece words as 16
// 32-bit words, `out[0..31]` receives the legal-target word of every slot.  Returns whether the
// side to move is in check.
__device__ __forceinline__ unsigned piece_word(const unsigned* my, int p) {
    return (my[p >> 1] >> (16 * (p & 1))) & 0xFFFFu;
}
__device__ __forceinline__ bool board_moves(const unsigned* my, bool black, unsigned long long* out) {
    // ---- pass 1: bitboards ----
    unsigned long long occ = 0, own = 0, e_pawns = 0, e_knights = 0, e_diag = 0, e_line = 0, e_king = 0;
    unsigned long long ep_pawns = 0, fresh_rooks = 0, my_king = 0;
    bool by_slot = true;                 // white in slots 0-15, black in 16-31, as the engine keeps them
#pragma unroll 1
    for (int p = 0; p < 32; ++p) {
        const unsigned word = piece_word(my, p);
        out[p] = 0ull;
        if ((word >> 11) & 1u) continue;
        const bool is_black = (word >> 10) & 1u, special = (word >> 9) & 1u;
        by_slot &= is_black == (p >= 16);
        const int type = (word >> 6) & 7;
        const unsigned long long bb = 1ull << (word & 63u);
        occ |= bb;
        if (is_black == black) {
            own |= bb;
            if (type == KING) my_king |= bb;
            if (type == ROOK && !special) fresh_rooks |= bb;
        } else {
            if (type == PAWN) { e_pawns |= bb; if (special) ep_pawns |= bb; }
            else if (type == KNIGHT) e_knights |= bb;
            else if (type == KING) e_king |= bb;
            else {
                if (type == BISHOP || type == QUEEN) e_diag |= bb;
                if (type == ROOK || type == QUEEN) e_line |= bb;
            }
        }
    }
    const unsigned long long opp = occ & ~own;
    const int king_sq = my_king ? __ffsll(static_cast<long long>(my_king)) - 1 : 0;
    // ---- what the opponent attacks, with the mover's king lifted off the board ----
    const unsigned long long occ_nk = occ & ~my_king;
    const unsigned long long danger = pawn_attacks(e_pawns, !black) | knight_pattern(e_knights) |
                                      king_pattern(e_king) | fill_diag(e_diag, occ_nk) | fill_line(e_line, occ_nk);
    // ---- checkers and the squares that answer a single check ----
    const unsigned long long kd_ex = diag_ex(king_sq), ka_ex = anti_ex(king_sq), kr_ex = rank_ex(king_sq),
                             kf_ex = file_ex(king_sq);
    const unsigned long long k_diag = line_attacks(my_king, occ, kd_ex) | line_attacks(my_king, occ, ka_ex);
    const unsigned long long k_line = line_attacks(my_king, occ, kr_ex) | line_attacks(my_king, occ, kf_ex);
    const unsigned long long checkers = (knight_pattern(my_king) & e_knights) | (pawn_attacks(my_king, black) & e_pawns) |
                                        (k_diag & e_diag) | (k_line & e_line);
    const bool chk = checkers != 0ull;
    unsigned long long target_mask = ~0ull;
    if (chk) {
        if (checkers & (checkers - 1ull)) target_mask = 0ull;               // two checkers: only the king moves
        else {
            unsigned long long between = 0ull;
            if (checkers & k_diag & e_diag) between = k_diag & piece_diag(checkers, occ);
            else if (checkers & k_line & e_line) between = k_line & piece_line(checkers, occ);
            target_mask = checkers | between;
        }
    }
    // ---- pieces that shield the king from a slider: the first own piece on a ray from the
    //      king, with an enemy slider of that ray's kind next behind it ----
    unsigned long long pinned = 0ull;
    if (my_king != 0ull) {
        const unsigned long long shields = (k_diag | k_line) & own;
        const unsigned long long occ2 = occ & ~shields;
        const unsigned long long k_diag2 = line_attacks(my_king, occ2, kd_ex) | line_attacks(my_king, occ2, ka_ex);
        const unsigned long long k_line2 = line_attacks(my_king, occ2, kr_ex) | line_attacks(my_king, occ2, kf_ex);
        for (unsigned long long pin = (k_diag2 & ~k_diag) & e_diag; pin != 0ull; pin &= pin - 1ull)
            pinned |= k_diag2 & piece_diag(pin & (0ull - pin), occ2) & shields;
        for (unsigned long long pin = (k_line2 & ~k_line) & e_line; pin != 0ull; pin &= pin - 1ull)
            pinned |= k_line2 & piece_line(pin & (0ull - pin), occ2) & shields;
    }
    // ---- the mover's pieces, one by one: its sixteen slots (all thirty-two for a board that
    //      does not keep the colours apart by slot) ----
    const int p_lo = by_slot ? (black ? 16 : 0) : 0, p_hi = by_slot ? p_lo + 16 : 32;
#pragma unroll 1
    for (int p = p_lo; p < p_hi; ++p) {
        const unsigned word = piece_word(my, p);
        if (((word >> 11) & 1u) || (((word >> 10) & 1u) != 0u) != black) continue;
        const bool special = (word >> 9) & 1u;
        const int type = (word >> 6) & 7, sq = word & 63;
        const int rank = sq >> 3, file = sq & 7;
        const unsigned long long bb = 1ull << sq;
        unsigned long long cand = 0ull, ep_target = 0ull;
        if (type == KING) {
            cand = king_pattern(bb) & ~danger;
            if (!special && !chk) {
                const int row = black ? 56 : 0;
                if ((fresh_rooks >> (row + 7)) & 1ull)
                    if (((occ >> (row + 5)) & 3ull) == 0ull && ((danger >> (row + 5)) & 3ull) == 0ull)
                        cand |= 1ull << (row + 6);
                if ((fresh_rooks >> row) & 1ull)
                    if (((occ >> (row + 1)) & 7ull) == 0ull && ((danger >> (row + 2)) & 3ull) == 0ull)
                        cand |= 1ull << (row + 2);
            }
            out[p] = cand & ~own;
            continue;
        }
        if (type == KNIGHT) {
            cand = knight_pattern(bb);
        } else if (type == PAWN) {
            const int up = black ? -8 : 8;
            const int f1 = sq + up;
            if (f1 >= 0 && f1 < 64) {
                if (!((occ >> f1) & 1ull)) {
                    cand |= 1ull << f1;
                    const bool start = black ? rank == 6 : rank == 1;
                    if (start && !((occ >> (f1 + up)) & 1ull)) cand |= 1ull << (f1 + up);
                }
                if (file > 0) cand |= (1ull << (f1 - 1)) & opp;
                if (file < 7) cand |= (1ull << (f1 + 1)) & opp;
                if (rank == (black ? 3 : 4)) {
                    if (file > 0 && ((ep_pawns >> (sq - 1)) & 1ull)) ep_target |= 1ull << (f1 - 1);
                    if (file < 7 && ((ep_pawns >> (sq + 1)) & 1ull)) ep_target |= 1ull << (f1 + 1);
                }
            }
        } else {
            if (type == BISHOP || type == QUEEN)
                cand |= line_attacks(bb, occ, diag_ex(sq)) | line_attacks(bb, occ, anti_ex(sq));
            if (type == ROOK || type == QUEEN)
                cand |= line_attacks(bb, occ, rank_ex(sq)) | line_attacks(bb, occ, file_ex(sq));
        }
        cand &= ~own;
        ep_target &= ~own;
        if (my_king == 0ull) { out[p] = cand | ep_target; continue; }       // no king to protect
        unsigned long long legal = cand & target_mask;
        if (bb & pinned) legal &= line_through(king_sq, sq);
        // en passant takes two pieces off one rank at once: tested on the position after it
        for (unsigned long long rest = ep_target; rest != 0ull; rest &= rest - 1ull) {
            const unsigned long long tb = rest & (0ull - rest);
            const unsigned long long gone = black ? tb << 8 : tb >> 8;
            const unsigned long long after = ((occ & ~bb) & ~gone) | tb;
            const bool hit = (knight_pattern(my_king) & e_knights) != 0ull ||
                             (pawn_attacks(my_king, black) & (e_pawns & ~gone)) != 0ull ||
                             (king_pattern(my_king) & e_king) != 0ull ||
                             ((line_attacks(my_king, after, kd_ex) | line_attacks(my_king, after, ka_ex)) & e_diag) != 0ull ||
                             ((line_attacks(my_king, after, kr_ex) | line_attacks(my_king, after, kf_ex)) & e_line) != 0ull;
            if (!hit) legal |= tb;
        }
        out[p] = legal;
    }
    return chk;
}

// Castling rights KQkq as four bits of a board held by one thread (torch_impl.py:294-318).
__device__ __forceinline__ unsigned board_rights(const unsigned* my) {
    bool wk = false, bk = false, k = false, q = false, k2 = false, q2 = false;
#pragma unroll 1
    for (int p = 0; p < 32; ++p) {
        const unsigned word = piece_word(my, p);
        if (((word >> 11) & 1u) || ((word >> 9) & 1u)) continue;
        const bool is_black = (word >> 10) & 1u;
        const int type = (word >> 6) & 7, sq = word & 63;
        if (type == KING) { if (is_black) bk = true; else wk = true; }
        if (type == ROOK) {
            if (!is_black) { k |= sq == 7; q |= sq == 0; }
            else { k2 |= sq == 63; q2 |= sq == 56; }
        }
    }
    return (wk && k ? 1u : 0u) | (wk && q ? 2u : 0u) | (bk && k2 ? 4u : 0u) | (bk && q2 ? 8u : 0u);
}
__device__ __forceinline__ void set_piece(unsigned* my, int p, unsigned v) {
    const int sh = 16 * (p & 1);
    my[p >> 1] = (my[p >> 1] & ~(0xFFFFu << sh)) | ((v & 0xFFFFu) << sh);
}
// Apply one move (`move` = slot * 64 + target, -1 = no move; `promo` 0..3 = N B R Q, negative =
// queen) to a board held by one thread: the reference's `step` without its hash
// (brokefish/env/torch_impl.py:412-548).  Capture: the first live piece on the target square, or
// for a pawn the en passant victim, which carries the double-step flag and stands beside the
// target's file neighbour, not on it.  `irreversible`: capture, pawn move or a change of
// castling rights.
__device__ __forceinline__ void board_step(unsigned* my, int control, int move, int promo, int& new_control,
                                           bool& irreversible) {
    new_control = control;
    irreversible = false;
    if (move < 0) return;
    const int source = move >> 6, target = move & 63;
    const bool white = control > 0;
    const unsigned mover = piece_word(my, source);
    const int mtype = (mover >> 6) & 7, from = mover & 63;
    const bool is_pawn = mtype == PAWN;
    const unsigned rights_before = board_rights(my);
    const unsigned victim_word = ((white ? 3u : 1u) << 9) + static_cast<unsigned>(target + (white ? -8 : 8));
    const int dx = target - from;
    const bool castling = mtype == KING && (dx == 2 || dx == -2);
    const int corner = (white ? 0 : 56) + (dx > 0 ? 7 : 0);
    int captured = -1, rook = -1;
#pragma unroll 1
    for (int p = 0; p < 32; ++p) {
        const unsigned word = piece_word(my, p);
        const bool live = ((word >> 11) & 1u) == 0u;
        if (captured < 0 && ((live && static_cast<int>(word & 63u) == target) || (is_pawn && word == victim_word)))
            captured = p;
    }
    if (captured >= 0) set_piece(my, captured, 1u << 11);
    // the corner rook is looked for by its square before anything moved, by its type after the capture
    if (castling) {
#pragma unroll 1
        for (int p = 0; p < 32; ++p) {
            const unsigned word = piece_word(my, p);
            const unsigned square = p == captured ? static_cast<unsigned>(target) : (word & 63u);
            if (rook < 0 && ((word >> 6) & 7u) == ROOK && static_cast<int>(square) == corner) rook = p;
        }
    }
    {
        unsigned w = (piece_word(my, source) & ~63u & 0xFFFu) + static_cast<unsigned>(target);
        if (is_pawn && (target >> 3) == (white ? 7 : 0))
            w += static_cast<unsigned>(promo < 0 ? QUEEN : promo + KNIGHT) << 6;
        if (mtype == KING || mtype == ROOK) w |= 1u << 9;
        set_piece(my, source, w);
    }
    if (rook >= 0)
        set_piece(my, rook, (piece_word(my, rook) & ~63u & 0xFFFu) + static_cast<unsigned>((white ? 0 : 56) + (dx > 0 ? 5 : 3)));
    // the en passant flag lives for one ply: clear every pawn's, set the double-stepper's
#pragma unroll 1
    for (int p = 0; p < 32; ++p) {
        const unsigned word = piece_word(my, p);
        if (((word >> 6) & 7u) == PAWN && ((word >> 9) & 1u)) set_piece(my, p, word & ~(1u << 9) & 0xFFFu);
    }
    if (is_pawn && (dx == 16 || dx == -16)) set_piece(my, source, piece_word(my, source) | (1u << 9));
    const int mag = (captured >= 0 || is_pawn) ? 1 : (control < 0 ? -control : control) + 1;
    new_control = white ? -mag : mag;
    irreversible = captured >= 0 || is_pawn || board_rights(my) != rights_before;
}

// Position keys.  The reference hashes a position with a table of random 64-bit keys indexed by
// (colour, type, square), side to move, the four castling rights and the file of a LEGAL en
// passant capture (brokefish/env/torch_impl.py:374-401, 321-371); only equality of hashes is
// ever used (repetition), so the keys here are this library's own: a 64-bit mix of the index.
__device__ __forceinline__ unsigned long long zobrist_key(int index) {
    unsigned long long x = 0x9E3779B97F4A7C15ull * static_cast<unsigned long long>(index + 1);
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
enum { ZOBRIST_SIDE = 768, ZOBRIST_CASTLE = 769, ZOBRIST_EP = 773 };

// Hash of a board held by one thread.  The en passant file counts only when a capture is really
// available: a pawn of the mover stands beside the pawn that has just made its double step, and
// taking it does not leave the mover's king attacked.
__device__ __forceinline__ unsigned long long board_hash(const unsigned* my, bool black) {
    unsigned long long h = black ? zobrist_key(ZOBRIST_SIDE) : 0ull;
    unsigned long long occ = 0, my_pawns = 0, my_king = 0, flagged = 0;
    unsigned long long e_pawns = 0, e_knights = 0, e_diag = 0, e_line = 0, e_king = 0;
#pragma unroll 1
    for (int p = 0; p < 32; ++p) {
        const unsigned word = piece_word(my, p);
        if ((word >> 11) & 1u) continue;
        const bool is_black = (word >> 10) & 1u, special = (word >> 9) & 1u;
        const int type = (word >> 6) & 7, sq = word & 63;
        const unsigned long long bb = 1ull << sq;
        h ^= zobrist_key(((is_black ? 6 : 0) + type) * 64 + sq);
        occ |= bb;
        if (is_black == black) {
            if (type == PAWN) my_pawns |= bb;
            if (type == KING) my_king |= bb;
        } else {
            if (type == PAWN) { e_pawns |= bb; if (special) flagged |= bb; }
            else if (type == KNIGHT) e_knights |= bb;
            else if (type == KING) e_king |= bb;
            else {
                if (type == BISHOP || type == QUEEN) e_diag |= bb;
                if (type == ROOK || type == QUEEN) e_line |= bb;
            }
        }
    }
    const unsigned rights = board_rights(my);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if ((rights >> i) & 1u) h ^= zobrist_key(ZOBRIST_CASTLE + i);
    if (flagged != 0ull) {
        const unsigned long long victim = flagged & (0ull - flagged);
        const int vsq = __ffsll(static_cast<long long>(victim)) - 1, vfile = vsq & 7;
        const unsigned long long target = black ? victim >> 8 : victim << 8;
        const int ksq = my_king ? __ffsll(static_cast<long long>(my_king)) - 1 : 0;
        bool legal = false;
#pragma unroll
        for (int side = 0; side < 2; ++side) {
            const unsigned long long capturer = side ? ((victim << 1) & ~kFileA) : ((victim >> 1) & ~kFileH);
            if ((capturer & my_pawns) == 0ull) continue;
            const unsigned long long after = ((occ & ~capturer) & ~victim) | target;
            const bool hit = my_king != 0ull &&
                             ((knight_pattern(my_king) & e_knights) != 0ull ||
                              (pawn_attacks(my_king, black) & (e_pawns & ~victim)) != 0ull ||
                              (king_pattern(my_king) & e_king) != 0ull ||
                              ((line_attacks(my_king, after, diag_ex(ksq)) | line_attacks(my_king, after, anti_ex(ksq))) & e_diag) != 0ull ||
                              ((line_attacks(my_king, after, rank_ex(ksq)) | line_attacks(my_king, after, file_ex(ksq))) & e_line) != 0ull);
            legal |= !hit;
        }
        if (legal) h ^= zobrist_key(ZOBRIST_EP + vfile);
    }
    return h;
}

// One thread per board, boards and legal words staged through shared memory for coalescing.
// `hash_out` non-null: the position key of the resulting board.
// kStep: play `move` first (or, with kPick, the floor(r * count)-th legal move of the incoming
// `mask` in (slot, square) order; a board without legal moves stays as it is) and write the new
// board, control word and irreversible flag; `mask` non-null: the legal words of the resulting
// board follow.  In place (boards_out == boards) is safe: a block reads all its boards first.
template <bool kStep, bool kPick>
__global__ void __launch_bounds__(kTpbThreads) engine_board_kernel(
        const uint16_t* __restrict__ boards, const int16_t* __restrict__ control, const int* __restrict__ move,
        const signed char* __restrict__ promo, const float* __restrict__ r, int n, uint16_t* boards_out,
        int16_t* control_out, unsigned char* __restrict__ irreversible, unsigned long long* mask,
        unsigned char* __restrict__ in_check, int* __restrict__ move_out, unsigned long long* __restrict__ hash_out) {
    extern __shared__ unsigned long long tpb_smem[];
    unsigned long long* s_out = tpb_smem;                                        // [128][33]
    unsigned* s_in = reinterpret_cast<unsigned*>(tpb_smem + kTpbThreads * kTpbOutStride);   // [128][17]
    const int tid = threadIdx.x;
    const long first = static_cast<long>(blockIdx.x) * kTpbThreads;
    const int here = static_cast<int>(min(static_cast<long>(kTpbThreads), n - first));
    {
        // coalesced load: the block's boards are one contiguous run of 16-byte pieces
        const uint4* src = reinterpret_cast<const uint4*>(boards + first * 32);
        for (int j = tid; j < here * 4; j += kTpbThreads) {
            const uint4 v = __ldg(src + j);
            unsigned* d = s_in + (j >> 2) * kTpbInStride + (j & 3) * 4;
            d[0] = v.x; d[1] = v.y; d[2] = v.z; d[3] = v.w;
        }
        if (kPick)
            for (int j = tid; j < here * 32; j += kTpbThreads)
                s_out[(j >> 5) * kTpbOutStride + (j & 31)] = mask[first * 32 + j];
    }
    __syncthreads();
    bool moved = false;
    if (tid < here) {
        unsigned* my = s_in + tid * kTpbInStride;
        unsigned long long* out = s_out + tid * kTpbOutStride;
        int ctl = control[first + tid];
        bool generate = mask != nullptr;
        if (kStep) {
            int mv = kPick ? -1 : move[first + tid];
            if (kPick) {
                int total = 0;
#pragma unroll 1
                for (int p = 0; p < 32; ++p) total += __popcll(out[p]);
                if (total > 0) {
                    int pick = static_cast<int>(__fmul_rn(r[first + tid], static_cast<float>(total)));
                    pick = pick < total - 1 ? pick : total - 1;
#pragma unroll 1
                    for (int p = 0; p < 32 && mv < 0; ++p) {
                        unsigned long long m = out[p];
                        const int cnt = __popcll(m);
                        if (pick < cnt) {
                            for (int i = 0; i < pick; ++i) m &= m - 1ull;
                            mv = p * 64 + __ffsll(static_cast<long long>(m)) - 1;
                        }
                        pick -= cnt;
                    }
                }
                if (move_out != nullptr) move_out[first + tid] = mv;
                generate = mv >= 0;                   // a finished game keeps its (empty) legal words
            }
            int nc;
            bool irr;
            board_step(my, ctl, mv, promo != nullptr ? promo[first + tid] : -1, nc, irr);
            moved = !kPick || mv >= 0;
            if (moved) {
                control_out[first + tid] = static_cast<int16_t>(nc);
                if (irreversible != nullptr) irreversible[first + tid] = irr ? 1 : 0;
            }
            ctl = nc;
        }
        if (generate) {
            const bool chk = board_moves(my, ctl < 0, out);
            if (in_check != nullptr) in_check[first + tid] = chk ? 1 : 0;
        }
        if (hash_out != nullptr) hash_out[first + tid] = board_hash(my, ctl < 0);
    }
    __syncthreads();
    if (kStep) {
        // coalesced store of the block's boards (all of them: a board that did not move is rewritten as it was)
        uint4* dst = reinterpret_cast<uint4*>(boards_out + first * 32);
        for (int j = tid; j < here * 4; j += kTpbThreads) {
            const unsigned* d = s_in + (j >> 2) * kTpbInStride + (j & 3) * 4;
            dst[j] = make_uint4(d[0], d[1], d[2], d[3]);
        }
    }
    if (mask != nullptr)
        for (int j = tid; j < here * 32; j += kTpbThreads)
            mask[first * 32 + j] = s_out[(j >> 5) * kTpbOutStride + (j & 31)];
}

// Why a game is over, one thread per board (brokefish/env/torch_impl.py:632-676): 1 checkmate,
// 2 stalemate (no legal move, with or without check), else 3 when the control word's magnitude
// has reached 101 (fifty moves without capture or pawn move), else 4 when the position has
// occurred three times (`rep_count`, from `repetition_kernel`; skipped when null), else 5 when
// neither side can mate -- no pawn, rook or queen and
// either no knight and every bishop on one colour of squares, or one knight and no bishop
// (torch_impl.py:604-629) -- else 0.  `result` is -1 for checkmate (the side to move lost), else 0.
__global__ void __launch_bounds__(128) terminal_kernel(const unsigned long long* __restrict__ mask,
                                                       const unsigned char* __restrict__ in_check,
                                                       const int16_t* __restrict__ control,
                                                       const uint16_t* __restrict__ boards,
                                                       const int* __restrict__ rep_count, int n,
                                                       unsigned char* __restrict__ code, signed char* __restrict__ result) {
    const long board = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (board >= n) return;
    unsigned long long any = 0ull;
    const ulonglong2* m2 = reinterpret_cast<const ulonglong2*>(mask + board * 32);
#pragma unroll 4
    for (int p = 0; p < 16; ++p) {
        const ulonglong2 v = __ldg(m2 + p);
        any |= v.x | v.y;
    }
    int heavy = 0, knights = 0, bishops = 0, dark = 0;
    const uint4* b4 = reinterpret_cast<const uint4*>(boards + board * 32);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const uint4 v = __ldg(b4 + q);
        const unsigned w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const unsigned word = (w[k >> 1] >> (16 * (k & 1))) & 0xFFFFu;
            if ((word >> 11) & 1u) continue;
            const int type = (word >> 6) & 7, sq = word & 63;
            heavy += type == PAWN || type == ROOK || type == QUEEN;
            knights += type == KNIGHT;
            bishops += type == BISHOP;
            dark += type == BISHOP && (((sq & 7) + (sq >> 3)) & 1) == 0;
        }
    }
    const int c = control[board];
    int out = 0;
    if (any == 0ull) out = in_check[board] ? 1 : 2;
    else if ((c < 0 ? -c : c) >= 101) out = 3;
    else if (rep_count != nullptr && rep_count[board] >= 3) out = 4;
    else if (heavy == 0 && ((knights == 0 && (dark == 0 || dark == bishops)) || (knights == 1 && bishops == 0))) out = 5;
    code[board] = static_cast<unsigned char>(out);
    if (result != nullptr) result[board] = out == 1 ? -1 : 0;
}

// The per-game repetition ring (brokefish/env/torch_impl.py:571-602): `ring` [n,100] position keys
// since the last irreversible move, `length` [n].  Push: record the position being left (`hash`
// is the key BEFORE the move, `irreversible` describes the move); an irreversible move empties
// the ring, because nothing at or before it can recur.
constexpr int kMaxHistory = 100;
__global__ void __launch_bounds__(128) history_push_kernel(unsigned long long* __restrict__ ring,
                                                           long long* __restrict__ length,
                                                           const unsigned long long* __restrict__ hash,
                                                           const unsigned char* __restrict__ irreversible, int n) {
    const long g = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= n) return;
    if (irreversible[g]) { length[g] = 0; return; }
    const long long len = length[g];
    ring[g * kMaxHistory + (len < kMaxHistory - 1 ? len : kMaxHistory - 1)] = hash[g];
    length[g] = len + 1 < kMaxHistory ? len + 1 : kMaxHistory;
}
// How many times the position has occurred, counting the present one.
__global__ void __launch_bounds__(128) repetition_kernel(const unsigned long long* __restrict__ hash,
                                                         const unsigned long long* __restrict__ ring,
                                                         const long long* __restrict__ length, int n,
                                                         int* __restrict__ count) {
    const long g = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (g >= n) return;
    const unsigned long long h = hash[g];
    long long len = length[g];
    len = len < kMaxHistory ? len : kMaxHistory;
    int c = 1;
    for (long long i = 0; i < len; ++i) c += ring[g * kMaxHistory + i] == h;
    count[g] = c;
}

}  // namespace bfmg
