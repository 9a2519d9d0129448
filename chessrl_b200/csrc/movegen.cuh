// Legal-move bitsets on the device, straight from the bit-packed input records (one thread per position).
// Replaces the per-position python-chess loop of the reference's callers (model_bis.py:373-380,
// Leela/pgn_to_input_data_decoder.py:35-42): bit m of a row = entry m of the 1858-move list is legal, in the
// mover's view (the record already shows the board from the side to move, which therefore always plays "up").
//
// Position recovered from a record: piece planes 0..11 of the newest history step, castling bytes, and the
// en-passant square from the previous step (their pawn left its start rank and stands two ranks further in the
// newest step - the only way that happens in one move is the double push). A record without history carries
// no en-passant right.
//
// Rules follow the library's host generator (chess.cpp): pseudo-legal moves, each tried on a copy of the board
// and kept when the mover's king is not attacked afterwards; castling needs the right, the rook on its corner,
// empty squares between, and king start / crossing squares not attacked (the landing square is covered by the
// general test). A knight promotion sets the bit of the plain from-to entry (model_bis.py:376-379).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>

namespace crl {

// 1..6 = mover's P N B R Q K, 7..12 = opponent's
__device__ __forceinline__ bool mg_theirs(int p) { return p >= 7; }
__device__ __forceinline__ bool mg_ours(int p) { return p >= 1 && p <= 6; }

__device__ bool mg_attacked(const int8_t* sq, int s) {   // by the opponent, who moves "down"
  const int f = s & 7, r = s >> 3;
  if (r < 7) {
    if (f > 0 && sq[(r + 1) * 8 + f - 1] == 7) return true;
    if (f < 7 && sq[(r + 1) * 8 + f + 1] == 7) return true;
  }
  const int kn[8][2] = {{1, 2}, {2, 1}, {2, -1}, {1, -2}, {-1, -2}, {-2, -1}, {-2, 1}, {-1, 2}};
  const int kg[8][2] = {{1, 0}, {1, 1}, {0, 1}, {-1, 1}, {-1, 0}, {-1, -1}, {0, -1}, {1, -1}};
  for (int i = 0; i < 8; ++i) {
    int nf = f + kn[i][0], nr = r + kn[i][1];
    if (nf >= 0 && nf < 8 && nr >= 0 && nr < 8 && sq[nr * 8 + nf] == 8) return true;
    nf = f + kg[i][0]; nr = r + kg[i][1];
    if (nf >= 0 && nf < 8 && nr >= 0 && nr < 8 && sq[nr * 8 + nf] == 12) return true;
  }
  for (int i = 0; i < 8; ++i) {      // kg[] doubles as the eight ray directions: odd = diagonal, even = straight
    const int df = kg[i][0], dr = kg[i][1];
    const int slider = (i & 1) ? 9 : 10;             // bishop on diagonals, rook on lines; queen on both
    int nf = f + df, nr = r + dr;
    while (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) {
      const int p = sq[nr * 8 + nf];
      if (p != 0) {
        if (p == slider || p == 11) return true;
        break;
      }
      nf += df; nr += dr;
    }
  }
  return false;
}

struct MoveGenParams {
  const uint8_t* recs;       // [batch, 840]
  long long batch;
  const short* plain_idx;    // [4096] from*64+to -> entry of the 1858 list (-1 where none)
  uint8_t* bits;             // [batch, stride]
  long long stride;          // >= 233
};

__global__ void __launch_bounds__(64) legal_mask_packed104_kernel(const MoveGenParams p) {
  const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= p.batch) return;
  const uint8_t* rec = p.recs + b * 840;
  int8_t sq[64];
  for (int s = 0; s < 64; ++s) sq[s] = 0;
  for (int pl = 0; pl < 12; ++pl)
    for (int r = 0; r < 8; ++r) {
      const unsigned byte = rec[pl * 8 + r];
      for (int f = 0; f < 8; ++f)
        if ((byte >> (7 - f)) & 1u) sq[r * 8 + f] = static_cast<int8_t>(pl + 1);
    }
  const bool ooo = rec[832] != 0, oo = rec[833] != 0;
  int ep = -1;
  {
    const unsigned now6 = rec[6 * 8 + 6], now4 = rec[6 * 8 + 4];        // their pawns, newest step: ranks 6 and 4
    const unsigned old6 = rec[19 * 8 + 6], old4 = rec[19 * 8 + 4];      // one step earlier (plane 13 + 6)
    const unsigned pushed = old6 & ~now6 & now4 & ~old4;
    for (int f = 0; f < 8; ++f)
      if ((pushed >> (7 - f)) & 1u) ep = 5 * 8 + f;
  }
  uint32_t bits[59];
  for (int i = 0; i < 59; ++i) bits[i] = 0u;
  int ksq = 0;
  for (int s = 0; s < 64; ++s)
    if (sq[s] == 6) ksq = s;

  // try a move on a copy; promo: 0 none, else the piece type placed (2..5)
  auto try_move = [&](int from, int to, int promo, bool is_ep, int castle_rook_from, int castle_rook_to) {
    int8_t c[64];
    for (int s = 0; s < 64; ++s) c[s] = sq[s];
    const int piece = c[from];
    if (is_ep) c[to - 8] = 0;
    c[to] = static_cast<int8_t>(promo ? promo : piece);
    c[from] = 0;
    if (castle_rook_from >= 0) { c[castle_rook_to] = c[castle_rook_from]; c[castle_rook_from] = 0; }
    const int k = piece == 6 ? to : ksq;
    if (mg_attacked(c, k)) return;
    int idx;
    if (promo >= 3) {                                   // q r b have their own entries after the 1792 plain ones
      const int f = from & 7, tf = to & 7;
      const int base = f == 0 ? 0 : 2 + 3 * (f - 1);
      const int rank = tf - (f == 0 ? 0 : f - 1);
      idx = 1792 + 3 * (base + rank) + (promo == 5 ? 0 : (promo == 4 ? 1 : 2));
    } else {
      idx = p.plain_idx[from * 64 + to];
    }
    if (idx >= 0 && idx < 1858) bits[idx >> 5] |= 1u << (idx & 31);
  };

  const int kn[8][2] = {{1, 2}, {2, 1}, {2, -1}, {1, -2}, {-1, -2}, {-2, -1}, {-2, 1}, {-1, 2}};
  const int kg[8][2] = {{1, 0}, {1, 1}, {0, 1}, {-1, 1}, {-1, 0}, {-1, -1}, {0, -1}, {1, -1}};
  for (int s = 0; s < 64; ++s) {
    const int pc = sq[s];
    if (!mg_ours(pc)) continue;
    const int f = s & 7, r = s >> 3;
    if (pc == 1) {
      if (r >= 7) continue;                              // no pawn stands on the last rank in a legal position
      const int one = s + 8;
      auto pawn_to = [&](int to, bool is_ep) {
        if (r == 6) { for (int pr = 5; pr >= 2; --pr) try_move(s, to, pr, false, -1, -1); }
        else try_move(s, to, 0, is_ep, -1, -1);
      };
      if (sq[one] == 0) {
        pawn_to(one, false);
        if (r == 1 && sq[one + 8] == 0) try_move(s, one + 8, 0, false, -1, -1);
      }
      for (int df = -1; df <= 1; df += 2) {
        const int nf = f + df;
        if (nf < 0 || nf > 7) continue;
        const int to = one + df;
        if (mg_theirs(sq[to])) pawn_to(to, false);
        else if (to == ep) pawn_to(to, true);
      }
    } else if (pc == 2 || pc == 6) {
      for (int i = 0; i < 8; ++i) {
        const int nf = f + (pc == 2 ? kn[i][0] : kg[i][0]), nr = r + (pc == 2 ? kn[i][1] : kg[i][1]);
        if (nf < 0 || nf > 7 || nr < 0 || nr > 7) continue;
        if (!mg_ours(sq[nr * 8 + nf])) try_move(s, nr * 8 + nf, 0, false, -1, -1);
      }
      if (pc == 6 && s == 4 && !mg_attacked(sq, 4)) {
        if (oo && sq[5] == 0 && sq[6] == 0 && sq[7] == 4 && !mg_attacked(sq, 5)) try_move(4, 6, 0, false, 7, 5);
        if (ooo && sq[3] == 0 && sq[2] == 0 && sq[1] == 0 && sq[0] == 4 && !mg_attacked(sq, 3)) try_move(4, 2, 0, false, 0, 3);
      }
    } else {
      for (int i = 0; i < 8; ++i) {
        if ((pc == 4 && (i & 1)) || (pc == 3 && !(i & 1))) continue;   // rook: lines only, bishop: diagonals only
        int nf = f + kg[i][0], nr = r + kg[i][1];
        while (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) {
          const int q = sq[nr * 8 + nf];
          if (q == 0) try_move(s, nr * 8 + nf, 0, false, -1, -1);
          else {
            if (mg_theirs(q)) try_move(s, nr * 8 + nf, 0, false, -1, -1);
            break;
          }
          nf += kg[i][0]; nr += kg[i][1];
        }
      }
    }
  }
  uint8_t* dst = p.bits + b * p.stride;
  for (int i = 0; i < 233; ++i) dst[i] = static_cast<uint8_t>(bits[i >> 2] >> ((i & 3) * 8));
}

}  // namespace crl
