"""Chess rules and input encoders of the reference, restated in plain Python (TEST INFRASTRUCTURE).

The reference leaves the rules to python-chess (unpinned third-party dependency, not installed here:
`chess.Board`, `legal_moves`, `mirror()`; call sites model_bis.py:373-380, utils/fen_encoder.py:5-38,
Leela/gen_TC.py:42-59,255-319, Leela/pgn_to_input_data_decoder.py:15-77). This module implements the
standard rules independently of the C++ library (dict board, generate-and-test legality) so that the two
can be compared move for move; both are also checked against the well-known perft node counts.

Encoders restated here:
* `planes19`  - utils/fen_encoder.py:5-38 (`[8,8,19]`, row 0 = rank 8).
* `planes112` - the server input: 8 history steps x (12 piece planes in the mover's view + 1 empty), then
  castling ours-OOO / ours-OO / theirs-OOO / theirs-OO, Black-to-move flag, two empty planes (the second
  optionally halfmove/100), ones (gen_TC.py:255-319, pgn_to_input_data_decoder.py:61-72, ustotheirs.py:4-23,
  read with the 102-plane meaning its comments state). Steps before the start of the game are empty.
* legal masks over the 1929 vocabulary (model_bis.py:373-380) and over the 1858 Leela entries from the
  mover's point of view (pgn_to_input_data_decoder.py:35-42).
"""
import numpy as np

from . import vocab

WHITE, BLACK = 0, 1
START_FEN = "rnbqkbnr/pppppppp/8/8/8/8/PPPPPPPP/RNBQKBNR w KQkq - 0 1"
KNIGHT = [(1, 2), (2, 1), (2, -1), (1, -2), (-1, -2), (-2, -1), (-2, 1), (-1, 2)]
KING = [(1, 0), (1, 1), (0, 1), (-1, 1), (-1, 0), (-1, -1), (0, -1), (1, -1)]
DIAG = [(1, 1), (1, -1), (-1, 1), (-1, -1)]
ORTH = [(1, 0), (-1, 0), (0, 1), (0, -1)]


class Position:
    """pieces: {(file, rank): symbol} with upper case = White."""

    def __init__(self, fen=START_FEN):
        parts = fen.split()
        self.pieces = {}
        for r, row in enumerate(parts[0].split("/")):
            f = 0
            for ch in row:
                if ch.isdigit():
                    f += int(ch)
                else:
                    self.pieces[(f, 7 - r)] = ch
                    f += 1
        self.turn = WHITE if parts[1] == "w" else BLACK
        self.castling = set(parts[2]) - {"-"}
        self.ep = None if parts[3] == "-" else ("abcdefgh".index(parts[3][0]), int(parts[3][1]) - 1)
        self.halfmove = int(parts[4]) if len(parts) > 4 else 0
        self.fullmove = int(parts[5]) if len(parts) > 5 else 1

    def copy(self):
        p = Position.__new__(Position)
        p.pieces, p.turn, p.castling, p.ep = dict(self.pieces), self.turn, set(self.castling), self.ep
        p.halfmove, p.fullmove = self.halfmove, self.fullmove
        return p

    @staticmethod
    def _mine(sym, side):
        return sym.isupper() == (side == WHITE)

    def attacked(self, sq, by):
        f, r = sq
        pawn, dr = ("P", -1) if by == WHITE else ("p", 1)
        for df in (-1, 1):
            if self.pieces.get((f + df, r + dr)) == pawn:
                return True
        for table, kinds in ((KNIGHT, "n"), (KING, "k")):
            for df, d in table:
                s = self.pieces.get((f + df, r + d))
                if s and s.lower() in kinds and self._mine(s, by):
                    return True
        for table, kinds in ((DIAG, "bq"), (ORTH, "rq")):
            for df, d in table:
                x, y = f + df, r + d
                while 0 <= x < 8 and 0 <= y < 8:
                    s = self.pieces.get((x, y))
                    if s:
                        if s.lower() in kinds and self._mine(s, by):
                            return True
                        break
                    x, y = x + df, y + d
        return False

    def king(self, side):
        k = "K" if side == WHITE else "k"
        return next(sq for sq, s in self.pieces.items() if s == k)

    def push(self, move):
        frm, to, promo = move
        sym = self.pieces.pop(frm)
        side = self.turn
        capture = to in self.pieces
        if sym.lower() == "p" and to == self.ep:
            del self.pieces[(to[0], frm[1])]
            capture = True
        self.pieces[to] = sym if not promo else (promo.upper() if side == WHITE else promo)
        if sym.lower() == "k" and abs(to[0] - frm[0]) == 2:
            rook_from, rook_to = ((7, frm[1]), (5, frm[1])) if to[0] == 6 else ((0, frm[1]), (3, frm[1]))
            self.pieces[rook_to] = self.pieces.pop(rook_from)
        self.ep = (frm[0], (frm[1] + to[1]) // 2) if sym.lower() == "p" and abs(to[1] - frm[1]) == 2 else None
        for sq in (frm, to):
            self.castling -= {(4, 0): {"K", "Q"}, (0, 0): {"Q"}, (7, 0): {"K"}, (4, 7): {"k", "q"}, (0, 7): {"q"},
                              (7, 7): {"k"}}.get(sq, set())
        self.halfmove = 0 if (sym.lower() == "p" or capture) else self.halfmove + 1
        if side == BLACK:
            self.fullmove += 1
        self.turn = 1 - side

    def pseudo(self):
        side = self.turn
        for (f, r), sym in list(self.pieces.items()):
            if not self._mine(sym, side):
                continue
            kind = sym.lower()
            if kind == "p":
                d, start, last = (1, 1, 6) if side == WHITE else (-1, 6, 1)
                targets = []
                if (f, r + d) not in self.pieces:
                    targets.append((f, r + d))
                    if r == start and (f, r + 2 * d) not in self.pieces:
                        yield ((f, r), (f, r + 2 * d), None)
                for df in (-1, 1):
                    t = (f + df, r + d)
                    if 0 <= t[0] < 8 and ((t in self.pieces and not self._mine(self.pieces[t], side)) or t == self.ep):
                        targets.append(t)
                for t in targets:
                    if r == last:
                        for pr in "qrbn":
                            yield ((f, r), t, pr)
                    else:
                        yield ((f, r), t, None)
            elif kind in "nk":
                for df, d in (KNIGHT if kind == "n" else KING):
                    t = (f + df, r + d)
                    if 0 <= t[0] < 8 and 0 <= t[1] < 8 and (t not in self.pieces or not self._mine(self.pieces[t], side)):
                        yield ((f, r), t, None)
                if kind == "k":
                    home = 0 if side == WHITE else 7
                    ks, qs, rook = ("K", "Q", "R") if side == WHITE else ("k", "q", "r")
                    if (f, r) == (4, home) and not self.attacked((4, home), 1 - side):
                        if ks in self.castling and (5, home) not in self.pieces and (6, home) not in self.pieces \
                                and self.pieces.get((7, home)) == rook and not self.attacked((5, home), 1 - side):
                            yield ((4, home), (6, home), None)
                        if qs in self.castling and all((x, home) not in self.pieces for x in (1, 2, 3)) \
                                and self.pieces.get((0, home)) == rook and not self.attacked((3, home), 1 - side):
                            yield ((4, home), (2, home), None)
            else:
                rays = (DIAG if kind in "bq" else []) + (ORTH if kind in "rq" else [])
                for df, d in rays:
                    x, y = f + df, r + d
                    while 0 <= x < 8 and 0 <= y < 8:
                        s = self.pieces.get((x, y))
                        if s is None:
                            yield ((f, r), (x, y), None)
                        else:
                            if not self._mine(s, side):
                                yield ((f, r), (x, y), None)
                            break
                        x, y = x + df, y + d

    def legal_moves(self):
        """Canonical order: by from-square, to-square (a1=0..h8=63), then promotion n < b < r < q."""
        out = []
        for m in self.pseudo():
            c = self.copy()
            c.push(m)
            if not c.attacked(c.king(self.turn), c.turn):
                out.append(m)
        rank = {None: 0, "n": 2, "b": 3, "r": 4, "q": 5}
        out.sort(key=lambda m: (m[0][1] * 8 + m[0][0], m[1][1] * 8 + m[1][0], rank[m[2]]))
        return out

    def mirror(self):
        """Ranks flipped, colours swapped (python-chess Board.mirror())."""
        m = self.copy()
        m.pieces = {(f, 7 - r): s.swapcase() for (f, r), s in self.pieces.items()}
        m.turn = 1 - self.turn
        m.castling = {c.swapcase() for c in self.castling}
        m.ep = None if self.ep is None else (self.ep[0], 7 - self.ep[1])
        return m

    def fen(self):
        rows = []
        for r in range(7, -1, -1):
            row, run = "", 0
            for f in range(8):
                s = self.pieces.get((f, r))
                if s is None:
                    run += 1
                else:
                    row += (str(run) if run else "") + s
                    run = 0
            rows.append(row + (str(run) if run else ""))
        cast = "".join(c for c in "KQkq" if c in self.castling) or "-"
        ep = "-" if self.ep is None else "abcdefgh"[self.ep[0]] + str(self.ep[1] + 1)
        return f"{'/'.join(rows)} {'wb'[self.turn]} {cast} {ep} {self.halfmove} {self.fullmove}"


def uci(move):
    (f0, r0), (f1, r1), promo = move
    return "abcdefgh"[f0] + str(r0 + 1) + "abcdefgh"[f1] + str(r1 + 1) + (promo or "")


def perft(pos, depth):
    moves = pos.legal_moves()
    if depth == 1:
        return len(moves)
    total = 0
    for m in moves:
        c = pos.copy()
        c.push(m)
        total += perft(c, depth - 1)
    return total


def planes19(pos):
    order = "PNBRQKpnbrqk"
    t = np.zeros((8, 8, 19), dtype=np.float32)
    for (f, r), s in pos.pieces.items():
        t[7 - r, f, order.index(s)] = 1.0
    t[:, :, 12] = 1.0 if pos.turn == WHITE else 0.0
    if pos.ep is not None:
        t[7 - pos.ep[1], pos.ep[0], 13] = 1.0
    for i, c in enumerate("KQkq"):
        t[:, :, 14 + i] = 1.0 if c in pos.castling else 0.0
    t[:, :, 18] = min(pos.halfmove / 100.0, 1.0)
    return t


def planes112(history, rule50=False):
    """history[0] = current position, history[1] = one ply earlier ...; returns [64, 112] f32 with token
    index rank*8+file of the board in the mover's view."""
    out = np.zeros((64, 112), dtype=np.float32)
    black = history[0].turn == BLACK
    order = "PNBRQKpnbrqk"
    for t, pos in enumerate(history[:8]):
        view = pos.mirror() if black else pos
        for (f, r), s in view.pieces.items():
            out[r * 8 + f, t * 13 + order.index(s)] = 1.0
    cur = history[0].mirror() if black else history[0]
    for i, c in enumerate("QKqk"):
        out[:, 104 + i] = 1.0 if c in cur.castling else 0.0
    out[:, 108] = 1.0 if black else 0.0
    if rule50:
        out[:, 109] = min(history[0].halfmove / 100.0, 1.0)
    out[:, 111] = 1.0
    return out


def legal_bits(pos, width):
    """uint8 bitset over the first `width` vocabulary entries (1929 or 1858); little-endian bit order."""
    lookup = {m: i for i, m in enumerate(vocab.policy_index)}
    flags = np.zeros(width, dtype=bool)
    for m in pos.legal_moves():
        idx = lookup[vocab.legal_token(uci(m))]
        if idx < width:
            flags[idx] = True
    return np.packbits(flags, bitorder="little")


class SplitMix64:
    def __init__(self, state):
        self.s = state & 0xFFFFFFFFFFFFFFFF

    def next(self):
        self.s = (self.s + 0x9E3779B97F4A7C15) & 0xFFFFFFFFFFFFFFFF
        z = self.s
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & 0xFFFFFFFFFFFFFFFF
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & 0xFFFFFFFFFFFFFFFF
        return z ^ (z >> 31)


def playout(seed, index, max_plies):
    """The seeded random playout that stands in for game data: plies ~ U{0..max_plies}, uniformly random
    legal moves from the start position (a finished game restarts). Returns the history, newest first."""
    mask = 0xFFFFFFFFFFFFFFFF
    rng = SplitMix64(((seed * 0x9E3779B97F4A7C15) + (index * 0xD1B54A32D192ED03) + 1) & mask)
    plies = rng.next() % (max_plies + 1)
    pos = Position()
    hist = [pos.copy()]
    for _ in range(plies):
        moves = pos.legal_moves()
        if not moves:
            pos = Position()
            hist = [pos.copy()]
            continue
        pos.push(moves[rng.next() % len(moves)])
        hist.append(pos.copy())
    if not pos.legal_moves():
        pos = Position()
        hist = [pos.copy()]
    return hist[::-1][:8]


def unpack_planes104(packed):
    """Test oracle for the "packed104" input layout: [B, 840] uint8 -> [B, 64, 112] float32 token-major planes.
    Bit order as the reference reads the lc0 record (LeelaData/show_value_head_ground_truth.py:70-86:
    `np.unpackbits` over the 8 bytes of a plane, square = 8*row + col), auxiliary bytes at the offsets of
    show_value_head_ground_truth.py:191-197 relative to the plane block (us_ooo, us_oo, them_ooo, them_oo,
    side to move, rule50 count)."""
    import numpy as np
    packed = np.asarray(packed, dtype=np.uint8)
    B = packed.shape[0]
    out = np.zeros((B, 64, 112), dtype=np.float32)
    bits = np.unpackbits(packed[:, :832], axis=1).reshape(B, 104, 64)
    out[:, :, :104] = bits.transpose(0, 2, 1)
    for k in range(4):
        out[:, :, 104 + k] = (packed[:, 832 + k] != 0)[:, None]
    out[:, :, 108] = (packed[:, 836] != 0)[:, None]
    out[:, :, 109] = np.minimum(packed[:, 837].astype(np.float32) / np.float32(100.0), np.float32(1.0))[:, None]
    out[:, :, 111] = 1.0
    return out


def pack_planes104(planes):
    """Inverse of `unpack_planes104` for representable planes ([B, 64, 112] float array) - numpy restatement used
    to cross-check the library's packer."""
    import numpy as np
    planes = np.asarray(planes, dtype=np.float32).reshape(-1, 64, 112)
    B = planes.shape[0]
    rec = np.zeros((B, 840), dtype=np.uint8)
    rec[:, :832] = np.packbits(planes[:, :, :104].transpose(0, 2, 1).reshape(B, 104 * 64) != 0, axis=1)
    for k in range(5):
        rec[:, 832 + k] = planes[:, 0, 104 + k] != 0
    rec[:, 837] = np.rint(planes[:, 0, 109].astype(np.float64) * 100.0).astype(np.uint8)
    return rec
