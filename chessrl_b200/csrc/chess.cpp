// Host-side chess rules for the inputs of the forward pass: legal-move generation, FEN parsing, the
// 19-plane encoding of utils/fen_encoder.py:5-38, the 112-plane history encoding the Leela server feeds
// (Leela/gen_TC.py:42-59,255-319 + Leela/pgn_to_input_data_decoder.py:61-72 + Leela/ustotheirs.py:4-23),
// the legal-move masks of model_bis.py:373-380 (1929 vocabulary) and pgn_to_input_data_decoder.py:35-42
// (1858 vocabulary, side-to-move perspective), and seeded random playouts from the start position.
// The reference delegates the rules to python-chess; this is an independent implementation, validated by
// perft node counts and against the Python restatement in the test oracle.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/chessrl_b200.h"
#include "vocab.h"

namespace {

enum { EMPTY = 0, WP = 1, WN, WB, WR, WQ, WK, BP, BN, BB, BR, BQ, BK };
enum { CWK = 1, CWQ = 2, CBK = 4, CBQ = 8 };

struct Move {
  int8_t from, to, promo;   // promo: 0 or piece type 2..5 (N, B, R, Q)
};

struct Board {
  int8_t sq[64];
  int8_t side;      // 0 white, 1 black
  int8_t castle;
  int8_t ep;        // en-passant target square or -1
  int16_t halfmove;
  int16_t fullmove;
};

inline int type_of(int p) { return p == 0 ? 0 : (p - 1) % 6 + 1; }        // 1..6 = P N B R Q K
inline int color_of(int p) { return p <= WK ? 0 : 1; }                    // only for p != 0
inline int file_of(int s) { return s & 7; }
inline int rank_of(int s) { return s >> 3; }

const int kKnight[8][2] = {{1, 2}, {2, 1}, {2, -1}, {1, -2}, {-1, -2}, {-2, -1}, {-2, 1}, {-1, 2}};
const int kKing[8][2] = {{1, 0}, {1, 1}, {0, 1}, {-1, 1}, {-1, 0}, {-1, -1}, {0, -1}, {1, -1}};
const int kDiag[4][2] = {{1, 1}, {1, -1}, {-1, 1}, {-1, -1}};
const int kOrth[4][2] = {{1, 0}, {-1, 0}, {0, 1}, {0, -1}};

void start_position(Board& b) {
  static const int8_t back[8] = {WR, WN, WB, WQ, WK, WB, WN, WR};
  std::memset(b.sq, 0, sizeof(b.sq));
  for (int f = 0; f < 8; ++f) {
    b.sq[f] = back[f];
    b.sq[8 + f] = WP;
    b.sq[48 + f] = BP;
    b.sq[56 + f] = static_cast<int8_t>(back[f] + 6);
  }
  b.side = 0; b.castle = CWK | CWQ | CBK | CBQ; b.ep = -1; b.halfmove = 0; b.fullmove = 1;
}

bool attacked(const Board& b, int s, int by) {
  const int f = file_of(s), r = rank_of(s);
  const int pawn = by == 0 ? WP : BP, knight = by == 0 ? WN : BN, king = by == 0 ? WK : BK;
  const int bishop = by == 0 ? WB : BB, rook = by == 0 ? WR : BR, queen = by == 0 ? WQ : BQ;
  const int pr = by == 0 ? r - 1 : r + 1;     // a pawn of `by` attacking s stands one rank behind it
  if (pr >= 0 && pr < 8) {
    if (f > 0 && b.sq[pr * 8 + f - 1] == pawn) return true;
    if (f < 7 && b.sq[pr * 8 + f + 1] == pawn) return true;
  }
  for (auto& d : kKnight) {
    const int nf = f + d[0], nr = r + d[1];
    if (nf >= 0 && nf < 8 && nr >= 0 && nr < 8 && b.sq[nr * 8 + nf] == knight) return true;
  }
  for (auto& d : kKing) {
    const int nf = f + d[0], nr = r + d[1];
    if (nf >= 0 && nf < 8 && nr >= 0 && nr < 8 && b.sq[nr * 8 + nf] == king) return true;
  }
  for (auto& d : kDiag) {
    int nf = f + d[0], nr = r + d[1];
    while (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) {
      const int p = b.sq[nr * 8 + nf];
      if (p != 0) { if (p == bishop || p == queen) return true; break; }
      nf += d[0]; nr += d[1];
    }
  }
  for (auto& d : kOrth) {
    int nf = f + d[0], nr = r + d[1];
    while (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) {
      const int p = b.sq[nr * 8 + nf];
      if (p != 0) { if (p == rook || p == queen) return true; break; }
      nf += d[0]; nr += d[1];
    }
  }
  return false;
}

int king_square(const Board& b, int side) {
  const int k = side == 0 ? WK : BK;
  for (int s = 0; s < 64; ++s) if (b.sq[s] == k) return s;
  return -1;
}

void make_move(Board& b, const Move& m) {
  const int p = b.sq[m.from], t = type_of(p), side = b.side;
  const int captured = b.sq[m.to];
  b.halfmove = (t == 1 || captured != 0) ? 0 : static_cast<int16_t>(b.halfmove + 1);
  if (t == 1 && m.to == b.ep) b.sq[side == 0 ? m.to - 8 : m.to + 8] = 0;        // en passant
  b.sq[m.to] = static_cast<int8_t>(p);
  b.sq[m.from] = 0;
  if (m.promo) b.sq[m.to] = static_cast<int8_t>(m.promo + (side == 0 ? 0 : 6));
  if (t == 6 && std::abs(m.to - m.from) == 2) {                                  // castling: move the rook
    if (m.to > m.from) { b.sq[m.from + 1] = b.sq[m.from + 3]; b.sq[m.from + 3] = 0; }
    else { b.sq[m.from - 1] = b.sq[m.from - 4]; b.sq[m.from - 4] = 0; }
  }
  b.ep = (t == 1 && std::abs(m.to - m.from) == 16) ? static_cast<int8_t>((m.from + m.to) / 2) : -1;
  auto clear = [&](int s) {
    if (s == 4) b.castle &= ~(CWK | CWQ);
    else if (s == 0) b.castle &= ~CWQ;
    else if (s == 7) b.castle &= ~CWK;
    else if (s == 60) b.castle &= ~(CBK | CBQ);
    else if (s == 56) b.castle &= ~CBQ;
    else if (s == 63) b.castle &= ~CBK;
  };
  clear(m.from); clear(m.to);
  if (side == 1) ++b.fullmove;
  b.side = static_cast<int8_t>(side ^ 1);
}

void pseudo_moves(const Board& b, std::vector<Move>& out) {
  const int side = b.side;
  for (int s = 0; s < 64; ++s) {
    const int p = b.sq[s];
    if (p == 0 || color_of(p) != side) continue;
    const int t = type_of(p), f = file_of(s), r = rank_of(s);
    auto add = [&](int to) { out.push_back({static_cast<int8_t>(s), static_cast<int8_t>(to), 0}); };
    if (t == 1) {
      const int dir = side == 0 ? 8 : -8, start = side == 0 ? 1 : 6, last = side == 0 ? 6 : 1;
      auto add_pawn = [&](int to) {
        if (r == last) for (int pr = 5; pr >= 2; --pr) out.push_back({static_cast<int8_t>(s), static_cast<int8_t>(to), static_cast<int8_t>(pr)});
        else add(to);
      };
      const int one = s + dir;
      if (b.sq[one] == 0) {
        add_pawn(one);
        if (r == start && b.sq[one + dir] == 0) add(one + dir);
      }
      for (int df = -1; df <= 1; df += 2) {
        const int nf = f + df;
        if (nf < 0 || nf > 7) continue;
        const int to = one + df;
        const int q = b.sq[to];
        if ((q != 0 && color_of(q) != side) || (to == b.ep && b.ep >= 0)) add_pawn(to);
      }
    } else if (t == 2 || t == 6) {
      const int (*tab)[2] = t == 2 ? kKnight : kKing;
      for (int i = 0; i < 8; ++i) {
        const int nf = f + tab[i][0], nr = r + tab[i][1];
        if (nf < 0 || nf > 7 || nr < 0 || nr > 7) continue;
        const int q = b.sq[nr * 8 + nf];
        if (q == 0 || color_of(q) != side) add(nr * 8 + nf);
      }
      if (t == 6) {
        const int home = side == 0 ? 4 : 60, ks = side == 0 ? CWK : CBK, qs = side == 0 ? CWQ : CBQ;
        const int rook = side == 0 ? WR : BR;
        if (s == home && !attacked(b, home, side ^ 1)) {
          if ((b.castle & ks) && b.sq[home + 1] == 0 && b.sq[home + 2] == 0 && b.sq[home + 3] == rook &&
              !attacked(b, home + 1, side ^ 1))
            add(home + 2);
          if ((b.castle & qs) && b.sq[home - 1] == 0 && b.sq[home - 2] == 0 && b.sq[home - 3] == 0 &&
              b.sq[home - 4] == rook && !attacked(b, home - 1, side ^ 1))
            add(home - 2);
        }
      }
    } else {
      for (int pass = 0; pass < 2; ++pass) {
        if ((pass == 0 && t == 4) || (pass == 1 && t == 3)) continue;    // rook: no diagonals, bishop: no lines
        const int (*tab)[2] = pass == 0 ? kDiag : kOrth;
        for (int i = 0; i < 4; ++i) {
          int nf = f + tab[i][0], nr = r + tab[i][1];
          while (nf >= 0 && nf < 8 && nr >= 0 && nr < 8) {
            const int q = b.sq[nr * 8 + nf];
            if (q == 0) add(nr * 8 + nf);
            else { if (color_of(q) != side) add(nr * 8 + nf); break; }
            nf += tab[i][0]; nr += tab[i][1];
          }
        }
      }
    }
  }
}

// legal moves in canonical order (from, to, promo ascending)
void legal_moves(const Board& b, std::vector<Move>& out) {
  std::vector<Move> pseudo;
  pseudo.reserve(64);
  pseudo_moves(b, pseudo);
  out.clear();
  for (const Move& m : pseudo) {
    Board c = b;
    make_move(c, m);
    if (!attacked(c, king_square(c, b.side), c.side)) out.push_back(m);
  }
  std::sort(out.begin(), out.end(), [](const Move& x, const Move& y) {
    if (x.from != y.from) return x.from < y.from;
    if (x.to != y.to) return x.to < y.to;
    return x.promo < y.promo;
  });
}

uint64_t perft(const Board& b, int depth) {
  std::vector<Move> moves;
  legal_moves(b, moves);
  if (depth == 1) return moves.size();
  uint64_t n = 0;
  for (const Move& m : moves) {
    Board c = b;
    make_move(c, m);
    n += perft(c, depth - 1);
  }
  return n;
}

bool parse_fen(const char* fen, Board& b) {
  std::memset(b.sq, 0, sizeof(b.sq));
  int r = 7, f = 0;
  const char* p = fen;
  static const char sym[] = " PNBRQKpnbrqk";
  for (; *p && *p != ' '; ++p) {
    if (*p == '/') { --r; f = 0; continue; }
    if (*p >= '1' && *p <= '8') { f += *p - '0'; continue; }
    const char* q = std::strchr(sym + 1, *p);
    if (q == nullptr || r < 0 || f > 7) return false;
    b.sq[r * 8 + f++] = static_cast<int8_t>(q - sym);
  }
  if (*p != ' ') return false;
  ++p;
  b.side = *p == 'b' ? 1 : 0;
  while (*p && *p != ' ') ++p;
  if (*p == ' ') ++p;
  b.castle = 0;
  for (; *p && *p != ' '; ++p) {
    if (*p == 'K') b.castle |= CWK; else if (*p == 'Q') b.castle |= CWQ;
    else if (*p == 'k') b.castle |= CBK; else if (*p == 'q') b.castle |= CBQ;
  }
  if (*p == ' ') ++p;
  b.ep = -1;
  if (*p && *p != '-' && p[1]) b.ep = static_cast<int8_t>((p[0] - 'a') + 8 * (p[1] - '1'));
  while (*p && *p != ' ') ++p;
  int hm = 0, fm = 1;
  if (*p) std::sscanf(p, "%d %d", &hm, &fm);
  b.halfmove = static_cast<int16_t>(hm);
  b.fullmove = static_cast<int16_t>(fm);
  return true;
}

std::string to_fen(const Board& b) {
  static const char sym[] = " PNBRQKpnbrqk";
  std::string s;
  for (int r = 7; r >= 0; --r) {
    int run = 0;
    for (int f = 0; f < 8; ++f) {
      const int p = b.sq[r * 8 + f];
      if (p == 0) { ++run; continue; }
      if (run) { s += static_cast<char>('0' + run); run = 0; }
      s += sym[p];
    }
    if (run) s += static_cast<char>('0' + run);
    if (r) s += '/';
  }
  s += b.side == 0 ? " w " : " b ";
  std::string c;
  if (b.castle & CWK) c += 'K';
  if (b.castle & CWQ) c += 'Q';
  if (b.castle & CBK) c += 'k';
  if (b.castle & CBQ) c += 'q';
  s += c.empty() ? "-" : c;
  s += ' ';
  if (b.ep >= 0) { s += static_cast<char>('a' + file_of(b.ep)); s += static_cast<char>('1' + rank_of(b.ep)); }
  else s += '-';
  s += ' ' + std::to_string(b.halfmove) + ' ' + std::to_string(b.fullmove);
  return s;
}

std::string uci(const Move& m) {
  std::string s;
  s += static_cast<char>('a' + file_of(m.from)); s += static_cast<char>('1' + rank_of(m.from));
  s += static_cast<char>('a' + file_of(m.to)); s += static_cast<char>('1' + rank_of(m.to));
  if (m.promo) s += " nbrq"[m.promo - 1];
  return s;
}

// rank-mirrored, colour-swapped copy (python-chess Board.mirror())
Board mirror(const Board& b) {
  Board m = b;
  for (int s = 0; s < 64; ++s) {
    const int p = b.sq[s ^ 56];
    m.sq[s] = static_cast<int8_t>(p == 0 ? 0 : (p <= WK ? p + 6 : p - 6));
  }
  m.side = static_cast<int8_t>(b.side ^ 1);
  m.castle = static_cast<int8_t>(((b.castle & (CWK | CWQ)) << 2) | ((b.castle & (CBK | CBQ)) >> 2));
  m.ep = b.ep >= 0 ? static_cast<int8_t>(b.ep ^ 56) : -1;
  return m;
}

int vocab_index(const std::string& token) {
  static const std::vector<std::pair<std::string, int>> sorted = [] {
    const crl::Vocab& v = crl::Vocab::get();
    std::vector<std::pair<std::string, int>> t;
    for (size_t i = 0; i < v.moves.size(); ++i) t.emplace_back(v.moves[i], static_cast<int>(i));
    std::sort(t.begin(), t.end());
    return t;
  }();
  auto it = std::lower_bound(sorted.begin(), sorted.end(), std::make_pair(token, -1));
  return (it != sorted.end() && it->first == token) ? it->second : -1;
}

// bit m set = vocabulary entry m is a legal move; knight promotions use the 4-character token
void legal_bits(const Board& b, uint8_t* bits, int nbytes) {
  std::memset(bits, 0, nbytes);
  std::vector<Move> moves;
  legal_moves(b, moves);
  for (const Move& m : moves) {
    std::string t = uci(m);
    if (t.size() == 5 && t[4] == 'n') t.pop_back();
    const int idx = vocab_index(t);
    if (idx >= 0 && idx / 8 < nbytes) bits[idx >> 3] |= static_cast<uint8_t>(1u << (idx & 7));
  }
}

void planes19(const Board& b, float* out) {     // [8][8][19], row 0 = rank 8 (fen_encoder.py:5-38)
  std::memset(out, 0, sizeof(float) * 64 * 19);
  for (int s = 0; s < 64; ++s) {
    const int p = b.sq[s];
    float* cell = out + ((7 - rank_of(s)) * 8 + file_of(s)) * 19;
    if (p) cell[p - 1] = 1.0f;
    cell[12] = b.side == 0 ? 1.0f : 0.0f;
    cell[14] = (b.castle & CWK) ? 1.0f : 0.0f;
    cell[15] = (b.castle & CWQ) ? 1.0f : 0.0f;
    cell[16] = (b.castle & CBK) ? 1.0f : 0.0f;
    cell[17] = (b.castle & CBQ) ? 1.0f : 0.0f;
    cell[18] = std::min(b.halfmove / 100.0f, 1.0f);
  }
  if (b.ep >= 0) out[((7 - rank_of(b.ep)) * 8 + file_of(b.ep)) * 19 + 13] = 1.0f;
}

// hist[0] = current position, hist[1] = one ply earlier, ... (n boards, n >= 1). out: [64][112] f32,
// token = rank*8+file of the board as seen by the side to move (mirrored when Black moves).
void planes112(const Board* hist, int n, int rule50, float* out) {
  std::memset(out, 0, sizeof(float) * 64 * 112);
  const bool black = hist[0].side == 1;
  for (int t = 0; t < 8 && t < n; ++t) {
    const Board v = black ? mirror(hist[t]) : hist[t];     // every step in the current mover's view
    for (int s = 0; s < 64; ++s) {
      const int p = v.sq[s];
      if (p) out[s * 112 + t * 13 + (p - 1)] = 1.0f;       // ours P..K then theirs; plane 12 of a step stays 0
    }
  }
  const Board cur = black ? mirror(hist[0]) : hist[0];
  for (int s = 0; s < 64; ++s) {
    float* cell = out + s * 112;
    cell[104] = (cur.castle & CWQ) ? 1.0f : 0.0f;          // ours O-O-O (ustotheirs.py:13)
    cell[105] = (cur.castle & CWK) ? 1.0f : 0.0f;          // ours O-O
    cell[106] = (cur.castle & CBQ) ? 1.0f : 0.0f;          // theirs O-O-O
    cell[107] = (cur.castle & CBK) ? 1.0f : 0.0f;          // theirs O-O
    cell[108] = black ? 1.0f : 0.0f;                       // 1 - colour
    cell[109] = rule50 ? std::min(hist[0].halfmove / 100.0f, 1.0f) : 0.0f;
    cell[111] = 1.0f;
  }
}

// One move in the notation the reference's callers use: SAN ("Nbd7", "exd6", "O-O-O", "cxb8=N+", as read by
// board.parse_san in Leela/pgn_to_input_data_decoder.py:24) or UCI ("g1f3", "c7b8n"). The text must select
// exactly one legal move.
bool parse_move_text(const Board& b, const std::string& text, Move& out) {
  std::string t = text;
  while (!t.empty() && (t.back() == '+' || t.back() == '#' || t.back() == '!' || t.back() == '?')) t.pop_back();
  if (t.empty()) return false;
  std::vector<Move> legal;
  legal_moves(b, legal);
  auto is_file = [](char c) { return c >= 'a' && c <= 'h'; };
  auto is_rank = [](char c) { return c >= '1' && c <= '8'; };
  if ((t.size() == 4 || t.size() == 5) && is_file(t[0]) && is_rank(t[1]) && is_file(t[2]) && is_rank(t[3])) {
    for (const Move& m : legal)
      if (uci(m) == t) { out = m; return true; }
    if (t.size() == 5) return false;         // four characters may still be SAN ("axb5" is not, but stay strict below)
  }
  int piece = 1, promo = 0, to = -1, from_file = -1, from_rank = -1;
  if (t == "O-O" || t == "0-0" || t == "O-O-O" || t == "0-0-0") {
    const int home = b.side == 0 ? 4 : 60;
    piece = 6; to = (t.size() == 3) ? home + 2 : home - 2; from_file = 4; from_rank = home >> 3;
  } else {
    size_t n = t.size();
    static const std::string kPieces = "NBRQK";
    if (n >= 2 && t[n - 2] == '=' && kPieces.find(t[n - 1]) != std::string::npos) { promo = static_cast<int>(kPieces.find(t[n - 1])) + 2; n -= 2; }
    else if (n >= 3 && kPieces.find(t[n - 1]) != std::string::npos && is_rank(t[n - 2])) { promo = static_cast<int>(kPieces.find(t[n - 1])) + 2; n -= 1; }
    if (promo == 6) return false;            // no promotion to a king
    if (n < 2 || !is_file(t[n - 2]) || !is_rank(t[n - 1])) return false;
    to = (t[n - 2] - 'a') + 8 * (t[n - 1] - '1');
    size_t i = 0;
    if (kPieces.find(t[0]) != std::string::npos) { piece = static_cast<int>(kPieces.find(t[0])) + 2; i = 1; }
    for (; i + 2 < n; ++i) {
      if (t[i] == 'x' || t[i] == '-') continue;
      if (is_file(t[i]) && from_file < 0) from_file = t[i] - 'a';
      else if (is_rank(t[i]) && from_rank < 0) from_rank = t[i] - '1';
      else return false;
    }
  }
  int found = 0;
  for (const Move& m : legal) {
    if (m.to != to || type_of(b.sq[m.from]) != piece || m.promo != promo) continue;
    if (from_file >= 0 && file_of(m.from) != from_file) continue;
    if (from_rank >= 0 && rank_of(m.from) != from_rank) continue;
    out = m;
    ++found;
  }
  return found == 1;
}

// hist[0] = current position, hist[1] = one ply earlier, ...: the packed record of planes112(hist, n, rule50)
// written directly (same planes, same bytes as crl_pack_planes104 of that tensor).
void pack_record(const Board* hist, int n, int rule50, uint8_t* rec) {
  std::memset(rec, 0, CRL_PACKED104_BYTES);
  const bool black = hist[0].side == 1;
  for (int t = 0; t < 8 && t < n; ++t) {
    const Board v = black ? mirror(hist[t]) : hist[t];
    for (int s = 0; s < 64; ++s)
      if (v.sq[s]) rec[(t * 13 + v.sq[s] - 1) * 8 + (s >> 3)] |= static_cast<uint8_t>(0x80u >> (s & 7));
  }
  const Board cur = black ? mirror(hist[0]) : hist[0];
  rec[832] = (cur.castle & CWQ) ? 1 : 0;
  rec[833] = (cur.castle & CWK) ? 1 : 0;
  rec[834] = (cur.castle & CBQ) ? 1 : 0;
  rec[835] = (cur.castle & CBK) ? 1 : 0;
  rec[836] = black ? 1 : 0;
  rec[837] = rule50 ? static_cast<uint8_t>(std::min<int>(hist[0].halfmove, 100)) : 0;
}

struct Rng {   // splitmix64
  uint64_t s;
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
};

uint16_t f32_to_f16(float f) {   // values here are 0, 1 or k/100: round-to-nearest-even
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  int32_t e = static_cast<int32_t>((x >> 23) & 0xff) - 127 + 15;
  uint32_t m = x & 0x7fffffu;
  if (e <= 0) {
    if (e < -10) return static_cast<uint16_t>(sign);
    m |= 0x800000u;
    const int shift = 14 - e;
    uint32_t h = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (h & 1))) ++h;
    return static_cast<uint16_t>(sign | h);
  }
  if (e >= 31) return static_cast<uint16_t>(sign | 0x7c00u);
  uint32_t h = (static_cast<uint32_t>(e) << 10) | (m >> 13);
  const uint32_t rem = m & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (h & 1))) ++h;
  return static_cast<uint16_t>(sign | h);
}

}  // namespace

extern "C" {

int crl_perft(const char* fen, int depth, uint64_t* nodes) {
  if (nodes == nullptr || depth < 1 || depth > 8) return CRL_ERR_INVALID;
  Board b;
  if (fen == nullptr) start_position(b);
  else if (!parse_fen(fen, b)) return CRL_ERR_INVALID;
  *nodes = perft(b, depth);
  return CRL_OK;
}

int crl_fen_to_planes19(const char* fen, float* out) {
  Board b;
  if (fen == nullptr || out == nullptr || !parse_fen(fen, b)) return CRL_ERR_INVALID;
  planes19(b, out);
  return CRL_OK;
}

int crl_successors(const char* fen, int32_t max_moves, char* ucis, char* fens, float* planes19_out, int32_t* count) {
  Board b;
  if (fen == nullptr || count == nullptr || max_moves < 0 || !parse_fen(fen, b)) return CRL_ERR_INVALID;
  std::vector<Move> moves;
  legal_moves(b, moves);
  *count = static_cast<int32_t>(moves.size());
  if (static_cast<int32_t>(moves.size()) > max_moves) return CRL_ERR_SHAPE;
  for (size_t i = 0; i < moves.size(); ++i) {
    Board c = b;
    make_move(c, moves[i]);
    if (ucis != nullptr) std::snprintf(ucis + i * 8, 8, "%s", uci(moves[i]).c_str());
    if (fens != nullptr) std::snprintf(fens + i * 96, 96, "%s", to_fen(c).c_str());
    if (planes19_out != nullptr) planes19(c, planes19_out + i * 64 * 19);
  }
  return CRL_OK;
}

int crl_legal_mask_1929(const char* fen, uint8_t* bits) {
  Board b;
  if (fen == nullptr || bits == nullptr || !parse_fen(fen, b)) return CRL_ERR_INVALID;
  legal_bits(b, bits, 242);
  return CRL_OK;
}

int crl_pack_planes104(const void* planes, int32_t layout, int64_t count, uint8_t* packed) {
  if (count < 0 || (count > 0 && (planes == nullptr || packed == nullptr))) return CRL_ERR_INVALID;
  if (layout != CRL_LAYOUT_NHWC_F16 && layout != CRL_LAYOUT_NHWC_F32) return CRL_ERR_INVALID;
  const bool f32 = layout == CRL_LAYOUT_NHWC_F32;
  // Every representable value is identified by its bit pattern: 0, 1, and c/100 for plane 109.
  auto bits_of = [&](float v) -> uint32_t {
    if (!f32) return f32_to_f16(v);
    uint32_t u;
    std::memcpy(&u, &v, 4);
    return u;
  };
  const uint32_t zero = bits_of(0.0f), one = bits_of(1.0f);
  uint32_t clock_bits[101];
  for (int c = 0; c <= 100; ++c) clock_bits[c] = bits_of(std::min(c / 100.0f, 1.0f));
  for (int64_t i = 0; i < count; ++i) {
    uint8_t* rec = packed + i * CRL_PACKED104_BYTES;
    std::memset(rec, 0, CRL_PACKED104_BYTES);
    auto at = [&](int s, int p) -> uint32_t {
      const size_t k = (static_cast<size_t>(i) * 64 + s) * 112 + p;
      if (f32) {
        uint32_t u;
        std::memcpy(&u, static_cast<const float*>(planes) + k, 4);
        return u == 0x80000000u ? 0u : u;                       // -0.0 counts as empty
      }
      const uint16_t h = static_cast<const uint16_t*>(planes)[k];
      return h == 0x8000u ? 0u : h;
    };
    for (int p = 0; p < 104; ++p)
      for (int s = 0; s < 64; ++s) {
        const uint32_t v = at(s, p);
        if (v == one) rec[p * 8 + (s >> 3)] |= static_cast<uint8_t>(0x80u >> (s & 7));
        else if (v != zero) return CRL_ERR_INVALID;
      }
    for (int p = 104; p < 112; ++p) {
      const uint32_t v = at(0, p);
      for (int s = 1; s < 64; ++s)
        if (at(s, p) != v) return CRL_ERR_INVALID;              // auxiliary planes are constant over the board
      if (p <= 108) {
        if (v != zero && v != one) return CRL_ERR_INVALID;
        rec[832 + (p - 104)] = v == one ? 1 : 0;
      } else if (p == 109) {
        int c = 0;
        while (c <= 100 && clock_bits[c] != v) ++c;
        if (c > 100) return CRL_ERR_INVALID;
        rec[837] = static_cast<uint8_t>(c);
      } else if (p == 110) {
        if (v != zero) return CRL_ERR_INVALID;
      } else if (v != one) {
        return CRL_ERR_INVALID;
      }
    }
  }
  return CRL_OK;
}

int crl_game_records(const char* moves, int32_t first_ply, int32_t count, int32_t rule50_plane, uint8_t* packed,
                     uint8_t* black, uint8_t* legal1858, char* fens, int32_t* bad_move) {
  if (bad_move != nullptr) *bad_move = -1;
  if (moves == nullptr || first_ply < 0 || count < 0) return CRL_ERR_INVALID;
  Board b;
  start_position(b);
  std::vector<Board> hist(1, b);
  std::vector<std::string> toks;
  {
    std::string cur;
    for (const char* p = moves;; ++p) {
      if (*p == ' ' || *p == '\t' || *p == '\n' || *p == 0) {
        if (!cur.empty()) { toks.push_back(cur); cur.clear(); }
        if (*p == 0) break;
      } else {
        cur += *p;
      }
    }
  }
  if (count > 0 && static_cast<size_t>(first_ply) + static_cast<size_t>(count) - 1 > toks.size()) return CRL_ERR_INVALID;
  auto emit = [&](int ply) {
    const int j = ply - first_ply;
    if (j < 0 || j >= count) return;
    std::vector<Board> recent(hist.rbegin(), hist.rbegin() + std::min<size_t>(8, hist.size()));
    if (packed != nullptr) pack_record(recent.data(), static_cast<int>(recent.size()), rule50_plane, packed + static_cast<size_t>(j) * CRL_PACKED104_BYTES);
    if (black != nullptr) black[j] = static_cast<uint8_t>(b.side);
    if (legal1858 != nullptr) legal_bits(b.side == 1 ? mirror(b) : b, legal1858 + static_cast<size_t>(j) * 233, 233);
    if (fens != nullptr) std::snprintf(fens + static_cast<size_t>(j) * 96, 96, "%s", to_fen(b).c_str());
  };
  emit(0);
  for (size_t i = 0; i < toks.size(); ++i) {
    Move m;
    if (!parse_move_text(b, toks[i], m)) {
      if (bad_move != nullptr) *bad_move = static_cast<int32_t>(i);
      return CRL_ERR_INVALID;
    }
    make_move(b, m);
    hist.push_back(b);
    emit(static_cast<int>(i) + 1);
  }
  return CRL_OK;
}

int crl_playout_positions(uint64_t seed, int64_t first, int64_t count, int32_t max_plies, int32_t rule50_plane,
                          uint16_t* planes112_f16, float* planes19_f32, uint8_t* legal1858, uint8_t* legal1929,
                          uint8_t* black, char* fens) {
  if (count < 0 || max_plies < 0 || max_plies > 1000) return CRL_ERR_INVALID;
  std::vector<float> tmp(64 * 112);
  std::vector<Move> moves;
  std::vector<Board> hist;
  for (int64_t i = 0; i < count; ++i) {
    Rng rng{seed * 0x9E3779B97F4A7C15ull + static_cast<uint64_t>(first + i) * 0xD1B54A32D192ED03ull + 1};
    const int plies = static_cast<int>(rng.next() % static_cast<uint64_t>(max_plies + 1));
    Board b;
    start_position(b);
    hist.assign(1, b);
    for (int ply = 0; ply < plies; ++ply) {
      legal_moves(b, moves);
      if (moves.empty()) {                   // mate or stalemate: start a new game, keep counting plies
        start_position(b);
        hist.assign(1, b);
        continue;
      }
      make_move(b, moves[rng.next() % moves.size()]);
      hist.push_back(b);
    }
    legal_moves(b, moves);
    if (moves.empty()) {                     // never emit a finished game
      start_position(b);
      hist.assign(1, b);
    }
    std::vector<Board> recent(hist.rbegin(), hist.rbegin() + std::min<size_t>(8, hist.size()));
    if (planes112_f16 != nullptr) {
      planes112(recent.data(), static_cast<int>(recent.size()), rule50_plane, tmp.data());
      uint16_t* dst = planes112_f16 + i * 64 * 112;
      for (int k = 0; k < 64 * 112; ++k) dst[k] = f32_to_f16(tmp[k]);
    }
    if (planes19_f32 != nullptr) planes19(b, planes19_f32 + i * 64 * 19);
    if (legal1858 != nullptr) legal_bits(b.side == 1 ? mirror(b) : b, legal1858 + i * 233, 233);
    if (legal1929 != nullptr) legal_bits(b, legal1929 + i * 242, 242);
    if (black != nullptr) black[i] = static_cast<uint8_t>(b.side);
    if (fens != nullptr) std::snprintf(fens + i * 96, 96, "%s", to_fen(b).c_str());
  }
  return CRL_OK;
}

}  // extern "C"
