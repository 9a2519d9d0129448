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
