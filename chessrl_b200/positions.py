"""Host-side input producers (library's own chess rules, see csrc/chess.cpp): FEN -> 19 planes, legal-move
masks, and the seeded random-playout position stream used as synthetic data (the reference's PGN / lc0
chunk data sets are not available offline)."""
import ctypes

import numpy as np
import torch

from . import _lib as L


def perft(fen, depth):
    n = ctypes.c_uint64(0)
    rc = L.load().crl_perft(fen.encode() if fen else None, depth, ctypes.byref(n))
    if rc != 0:
        raise L.CrlError(rc, "perft")
    return n.value


def fen_to_tensor(fen):
    """utils/fen_encoder.py:5-38: [8, 8, 19] float32 numpy array."""
    out = np.zeros((8, 8, 19), dtype=np.float32)
    rc = L.load().crl_fen_to_planes19(fen.encode(), out.ctypes.data)
    if rc != 0:
        raise L.CrlError(rc, f"bad FEN {fen!r}")
    return out


def fen_to_planes112(fen, rule50_plane=False):
    """One FEN -> [8, 8, 112] float16 planes of the 112-plane networks in the mover's view with an EMPTY history
    (only the newest of the eight board slots is filled): 12 piece planes (mover's P N B R Q K, then the
    opponent's; board rank-mirrored when Black is to move), castling planes 104..107 (ours O-O-O, ours O-O, theirs
    O-O-O, theirs O-O), plane 108 = Black to move, plane 109 = halfmove/100 if `rule50_plane`, plane 111 = ones -
    the plane semantics of Leela/gen_TC.py:42-59, 255-319 and Leela/ustotheirs.py:4-23. A FEN carries no earlier
    boards, so slots 1..7 stay empty, as for the first position of a game."""
    t = fen_to_tensor(fen)                            # [8, 8, 19], row 0 = rank 8, white pieces first
    black = t[0, 0, 12] == 0.0
    out = np.zeros((8, 8, 112), dtype=np.float16)
    if black:
        out[:, :, 0:6] = t[:, :, 6:12]                # mirrored ranks: row r of the view is row r of the rank-8-first tensor
        out[:, :, 6:12] = t[:, :, 0:6]
        cast = (t[0, 0, 17], t[0, 0, 16], t[0, 0, 15], t[0, 0, 14])     # q k Q K
    else:
        out[:, :, 0:12] = t[::-1, :, 0:12]
        cast = (t[0, 0, 15], t[0, 0, 14], t[0, 0, 17], t[0, 0, 16])     # Q K q k
    for i, c in enumerate(cast):
        out[:, :, 104 + i] = c
    out[:, :, 108] = 1.0 if black else 0.0
    if rule50_plane:
        out[:, :, 109] = t[0, 0, 18]
    out[:, :, 111] = 1.0
    return out


def mirror_uci(uci):
    """Rank-mirror a UCI move string (e2e4 <-> e7e5): the change of view between White's and Black's board."""
    return "".join(str(9 - int(c)) if c.isdigit() else c for c in uci)


def mirror_fen(fen):
    """The same position seen from the other side: ranks flipped, colours, side to move, castling rights and the
    en-passant square swapped with them."""
    f = fen.split()
    board = "/".join(r.swapcase() for r in reversed(f[0].split("/")))
    side = "w" if f[1] == "b" else "b"
    cast = "".join(sorted(f[2].swapcase(), key="KQkq".index)) if f[2] != "-" else "-"
    ep = mirror_uci(f[3]) if f[3] != "-" else "-"
    return " ".join([board, side, cast, ep] + f[4:])


def vocab_move(index):
    """Entry `index` of the reference's 1929-move policy vocabulary (utils/vocab.py `policy_index`) as a UCI string."""
    buf = ctypes.create_string_buffer(16)
    rc = L.load().crl_vocab_move(int(index), buf)
    if rc != 0:
        raise L.CrlError(rc, f"vocabulary index {index}")
    return buf.value.decode()


def legal_mask_1929(fen):
    """uint8 bitset [242] over the 1929 vocabulary (bit m little-endian in byte m//8)."""
    out = np.zeros(242, dtype=np.uint8)
    rc = L.load().crl_legal_mask_1929(fen.encode(), out.ctypes.data)
    if rc != 0:
        raise L.CrlError(rc, f"bad FEN {fen!r}")
    return out


def playout_positions(count, seed=20240607, first=0, max_plies=80, rule50_plane=True, planes112=True, planes19=False,
                      fens=False, pin_memory=False):
    """Seeded random-playout positions. Returns a dict of torch tensors: planes112 [count,8,8,112] f16 (token
    order a1..h8 in the mover's view), planes19 [count,8,8,19] f32, legal1858 [count,233] u8, legal1929
    [count,242] u8, black [count] u8 and (optionally) the FEN strings."""
    out = {}
    kw = dict(pin_memory=pin_memory)
    p112 = torch.empty(count, 8, 8, 112, dtype=torch.float16, **kw) if planes112 else None
    p19 = torch.empty(count, 8, 8, 19, dtype=torch.float32, **kw) if planes19 else None
    l1858 = torch.empty(count, 233, dtype=torch.uint8, **kw)
    l1929 = torch.empty(count, 242, dtype=torch.uint8, **kw)
    black = torch.empty(count, dtype=torch.uint8, **kw)
    fbuf = ctypes.create_string_buffer(96 * count) if fens else None
    rc = L.load().crl_playout_positions(seed, first, count, max_plies, int(rule50_plane),
                                        p112.data_ptr() if planes112 else None, p19.data_ptr() if planes19 else None,
                                        l1858.data_ptr(), l1929.data_ptr(), black.data_ptr(),
                                        ctypes.addressof(fbuf) if fens else None)
    if rc != 0:
        raise L.CrlError(rc, "playout_positions")
    if planes112:
        out["planes112"] = p112
    if planes19:
        out["planes19"] = p19
    out.update(legal1858=l1858, legal1929=l1929, black=black)
    if fens:
        out["fens"] = [fbuf.raw[i * 96:(i + 1) * 96].split(b"\0", 1)[0].decode() for i in range(count)]
    return out


def pack_planes104(planes, pin_memory=False):
    """[..., 8, 8, 112] f16/f32 host planes (token-major, as `playout_positions` yields them) -> [B, 840] uint8
    records of the "packed104" input layout: 104 bit planes in the byte/bit order of the lc0 training record
    (LeelaData/show_value_head_ground_truth.py:58-88) followed by castling, side-to-move and half-move-clock bytes.
    17 times fewer bytes to move to the GPU than f16 planes; the engine expands them on the device."""
    planes = planes.contiguous()
    if planes.device.type != "cpu" or planes.shape[-1] != 112 or planes.numel() % (64 * 112) != 0:
        raise ValueError("expected host planes [..., 8, 8, 112]")
    layout = {torch.float16: L.LAYOUT_NHWC_F16, torch.float32: L.LAYOUT_NHWC_F32}.get(planes.dtype)
    if layout is None:
        raise ValueError("planes must be float16 or float32")
    count = planes.numel() // (64 * 112)
    out = torch.empty(count, L.PACKED104_BYTES, dtype=torch.uint8, pin_memory=pin_memory)
    rc = L.load().crl_pack_planes104(planes.data_ptr(), layout, count, out.data_ptr())
    if rc != 0:
        raise L.CrlError(rc, "pack_planes104: a plane is not representable (piece planes 0/1, constant auxiliary planes)")
    return out


def game_records(moves, first_ply=0, count=None, rule50_plane=True, legal=False, fens=False, pin_memory=False):
    """Replay a game given as SAN or UCI move strings (the reference's `list_uci_to_input`,
    Leela/pgn_to_input_data_decoder.py:14-78, parses SAN) and return packed records for the positions after
    first_ply .. first_ply+count-1 moves, each with its history of up to 8 boards: dict with `packed` [count,840] u8,
    `black` [count] u8 and optionally `legal1858` [count,233] and `fens`. Raises ValueError naming the first token
    that does not select exactly one legal move."""
    moves = list(moves)
    if count is None:
        count = len(moves) + 1 - first_ply
    text = " ".join(moves).encode()
    packed = torch.empty(count, L.PACKED104_BYTES, dtype=torch.uint8, pin_memory=pin_memory)
    black = torch.empty(count, dtype=torch.uint8, pin_memory=pin_memory)
    lg = torch.empty(count, 233, dtype=torch.uint8, pin_memory=pin_memory) if legal else None
    fbuf = ctypes.create_string_buffer(96 * max(count, 1)) if fens else None
    bad = ctypes.c_int32(-1)
    rc = L.load().crl_game_records(text, first_ply, count, int(rule50_plane), packed.data_ptr(), black.data_ptr(),
                                   lg.data_ptr() if legal else None, ctypes.addressof(fbuf) if fens else None,
                                   ctypes.addressof(bad))
    if rc != 0:
        if bad.value >= 0:
            raise ValueError(f"move {bad.value} ({moves[bad.value]!r}) does not select exactly one legal move")
        raise L.CrlError(rc, "game_records")
    out = {"packed": packed, "black": black}
    if legal:
        out["legal1858"] = lg
    if fens:
        out["fens"] = [fbuf.raw[i * 96:(i + 1) * 96].split(b"\0", 1)[0].decode() for i in range(count)]
    return out


def successors(fen, planes19=True, pin_memory=False):
    """Legal moves of `fen` (UCI strings, ordered by from-square, to-square, promotion) with the FENs and, optionally,
    the 19-plane encodings [n,8,8,19] of the positions they lead to - the push / fen / pop loop of
    calculate_move_values (new_paradigm/value.py:330-340) in one library call."""
    n_max = 256
    ubuf = ctypes.create_string_buffer(8 * n_max)
    fbuf = ctypes.create_string_buffer(96 * n_max)
    planes = torch.empty(n_max, 8, 8, 19, dtype=torch.float32, pin_memory=pin_memory) if planes19 else None
    count = ctypes.c_int32(0)
    rc = L.load().crl_successors(fen.encode(), n_max, ctypes.addressof(ubuf), ctypes.addressof(fbuf),
                                 planes.data_ptr() if planes19 else None, ctypes.addressof(count))
    if rc != 0:
        raise L.CrlError(rc, "successors")
    n = count.value
    ucis = [ubuf.raw[i * 8:(i + 1) * 8].split(b"\0", 1)[0].decode() for i in range(n)]
    fens = [fbuf.raw[i * 96:(i + 1) * 96].split(b"\0", 1)[0].decode() for i in range(n)]
    return ucis, fens, (planes[:n] if planes19 else None)
