"""Chess rules and input encoders (no GPU): the library's C++ implementation and the oracle's independent
Python restatement against the well-known perft node counts, and against each other position by position
(moves, FENs, 19 planes, 112 planes, legal-move bitsets: all exact)."""
import numpy as np
import pytest

from oracle import chesspos, vocab

KIWIPETE = "r3k2r/p1ppqpb1/bn2pnp1/3PN3/1p2P3/2N2Q1p/PPPBBPPP/R3K2R w KQkq - 0 1"
ENDGAME = "8/2p5/3p4/KP5r/1R3p1k/8/4P1P1/8 w - - 0 1"
PROMO = "r3k2r/Pppp1ppp/1b3nbN/nP6/BBP1P3/q4N2/Pp1P2PP/R2Q1RK1 w kq - 0 1"


@pytest.mark.parametrize("fen,counts", [
    (None, [20, 400, 8902, 197281]),
    (KIWIPETE, [48, 2039, 97862]),
    (ENDGAME, [14, 191, 2812, 43238]),
    (PROMO, [6, 264, 9467]),
])
def test_library_perft(lib, fen, counts):
    from chessrl_b200 import positions
    for depth, want in enumerate(counts, start=1):
        assert positions.perft(fen, depth) == want


def test_library_perft_depth5_start(lib):
    from chessrl_b200 import positions
    assert positions.perft(None, 5) == 4865609


@pytest.mark.parametrize("fen,counts", [
    (chesspos.START_FEN, [20, 400, 8902]),
    (KIWIPETE, [48, 2039]),
    (ENDGAME, [14, 191, 2812]),
    (PROMO, [6, 264]),
])
def test_oracle_perft(fen, counts):
    for depth, want in enumerate(counts, start=1):
        assert chesspos.perft(chesspos.Position(fen), depth) == want


def test_playouts_planes_and_masks_match_oracle(lib):
    from chessrl_b200 import positions
    n, seed = 160, 20240607
    got = positions.playout_positions(n, seed=seed, max_plies=80, planes19=True, fens=True)
    p112 = got["planes112"].float().numpy().reshape(n, 64, 112)
    for i in range(n):
        hist = chesspos.playout(seed, i, 80)
        cur = hist[0]
        assert got["fens"][i] == cur.fen()
        assert int(got["black"][i]) == cur.turn
        np.testing.assert_array_equal(got["planes19"][i].numpy(), chesspos.planes19(cur))
        want112 = chesspos.planes112(hist, rule50=True)
        np.testing.assert_array_equal(p112[i], want112.astype(np.float16).astype(np.float32))
        np.testing.assert_array_equal(got["legal1929"][i].numpy(), chesspos.legal_bits(cur, 1929))
        view = cur.mirror() if cur.turn == chesspos.BLACK else cur
        np.testing.assert_array_equal(got["legal1858"][i].numpy(), chesspos.legal_bits(view, 1858))
    plies = [len(chesspos.playout(seed, i, 80)) for i in range(40)]
    assert min(plies) < 8 <= max(plies)           # short games (empty history steps) and full histories both occur


def test_fen_entry_points(lib):
    from chessrl_b200 import positions
    for fen in (chesspos.START_FEN, KIWIPETE, PROMO, "rnbqkbnr/pppp1ppp/8/4p3/4P3/8/PPPP1PPP/RNBQKBNR w KQkq e6 3 2"):
        pos = chesspos.Position(fen)
        np.testing.assert_array_equal(positions.fen_to_tensor(fen), chesspos.planes19(pos))
        np.testing.assert_array_equal(positions.legal_mask_1929(fen), chesspos.legal_bits(pos, 1929))
    # knight promotion folds onto the 4-character token (model_bis.py:376-379)
    bits = np.unpackbits(positions.legal_mask_1929(PROMO), bitorder="little")
    assert bits[vocab.policy_index.index("b7b8")] == 1 or bits[vocab.policy_index.index("a7a8")] == 0
    with pytest.raises(Exception):
        positions.fen_to_tensor("not a fen")


def test_mirror_symmetry_of_legal_moves():
    # legal(pos) <-> legal(mirror(pos)) under the rank-mirror of the move strings (compare_policy.py:437-463)
    for i in range(30):
        pos = chesspos.playout(7, i, 60)[0]
        a = sorted(vocab.mirror_uci(chesspos.uci(m)) for m in pos.legal_moves())
        b = sorted(chesspos.uci(m) for m in pos.mirror().legal_moves())
        assert a == b


def test_packed104_records_round_trip_and_reject_unrepresentable_planes(lib):
    """The bit-packed input records: library packer == the oracle's numpy packer byte for byte, the oracle's
    reading of the records (the bit order of the reference's lc0-record reader) gives back the planes exactly,
    the piece of the record the reference decodes (first 12 planes -> board) is the position's own board, and
    planes that cannot be represented are refused."""
    import torch
    from chessrl_b200 import positions, CrlError
    n = 300
    got = positions.playout_positions(n, seed=7, max_plies=120, fens=True)
    planes = got["planes112"]
    rec = positions.pack_planes104(planes)
    assert rec.shape == (n, 840) and rec.dtype == torch.uint8
    ref = planes.float().numpy().reshape(n, 64, 112)
    np.testing.assert_array_equal(rec.numpy(), chesspos.pack_planes104(ref))
    back = chesspos.unpack_planes104(rec.numpy())
    np.testing.assert_array_equal(back.astype(np.float16).astype(np.float32), ref)
    # the reference's reader: unpackbits over the first 96 bytes, square = 8*row + col, "PNBRQKpnbrqk"
    for i in range(0, n, 17):
        bits = np.unpackbits(rec[i, :96].numpy()).reshape(12, 64)
        board = [["." for _ in range(8)] for _ in range(8)]
        for k, ch in enumerate("PNBRQKpnbrqk"):
            for sq in np.nonzero(bits[k])[0]:
                board[7 - sq // 8][sq % 8] = ch
        pos = chesspos.Position(got["fens"][i])
        view = pos.mirror() if pos.turn == chesspos.BLACK else pos
        want = view.fen().split()[0]
        rows = []
        for r in board:
            out, run = "", 0
            for ch in r:
                if ch == ".":
                    run += 1
                else:
                    out += (str(run) if run else "") + ch
                    run = 0
            rows.append(out + (str(run) if run else ""))
        assert "/".join(rows) == want
        assert int(rec[i, 836]) == int(got["black"][i])
    # empty and ragged inputs, then planes with no packed form
    assert positions.pack_planes104(planes[:0]).shape == (0, 840)
    assert torch.equal(positions.pack_planes104(planes[5:6]), rec[5:6])
    for plane, tok, val in [(3, 10, 0.5), (104, 7, 1.0 - float(planes[0, 0, 7, 104])), (110, 0, 1.0), (111, 63, 0.0), (109, 1, 0.123)]:
        bad = planes[:2].clone()
        bad.view(2, 64, 112)[1, tok, plane] = val
        with pytest.raises(CrlError):
            positions.pack_planes104(bad)
    f32_exact = planes[:4].float()
    f32_exact.view(4, 64, 112)[:, :, 109] = torch.tensor([0.0, 0.07, 0.5, 1.0]).view(4, 1)
    assert positions.pack_planes104(f32_exact)[:, 837].tolist() == [0, 7, 50, 100]


def test_successors_match_oracle(lib):
    """Legal moves, resulting FENs and their 19-plane encodings of crl_successors against the oracle's rules, on
    positions with promotions, castling, en passant, check and mate."""
    from chessrl_b200 import positions
    fens = [chesspos.START_FEN, KIWIPETE, ENDGAME, PROMO,
            "rnbqkbnr/ppp1pppp/8/8/3pP3/8/PPPP1PPP/RNBQKBNR b KQkq e3 0 2",
            "1n1Rkb1r/p4ppp/4q3/4p1B1/4P3/8/PPP2PPP/2K5 b k - 1 17"]
    for fen in fens:
        ucis, nxt, planes = positions.successors(fen)
        pos = chesspos.Position(fen)
        want = {}
        for m in pos.legal_moves():
            c = pos.copy()
            c.push(m)
            want[chesspos.uci(m)] = c
        assert sorted(ucis) == sorted(want) and len(set(ucis)) == len(ucis)
        assert planes.shape == (len(ucis), 8, 8, 19)
        for u, f, p in zip(ucis, nxt, planes):
            assert f == want[u].fen()
            np.testing.assert_array_equal(p.numpy(), chesspos.planes19(want[u]))
    assert positions.successors(fens[-1])[0] == []          # mate: nothing to choose from
