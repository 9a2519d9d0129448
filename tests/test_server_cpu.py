"""Game replay (SAN / UCI -> packed records) and the policy server's wire protocol, without a GPU: the C++ replay
against the oracle's independent Python rules, the length-prefixed pickle framing and request pooling against a
stand-in engine, and the refusal of pickles that reference any global."""
import os
import pickle
import threading

import numpy as np
import pytest
import torch

from oracle import chesspos

# a nineteenth-century miniature: captures, checks, a file disambiguation, long castling, mate
SAN_A = ("e4 e5 Nf3 d6 d4 Bg4 dxe5 Bxf3 Qxf3 dxe5 Bc4 Nf6 Qb3 Qe7 Nc3 c6 Bg5 b5 Nxb5 cxb5 Bxb5+ Nbd7 O-O-O Rd8 "
         "Rxd7 Rxd7 Rd1 Qe6 Bxd7+ Nxd7 Qb8+ Nxb8 Rd8#").split()
UCI_A = ("e2e4 e7e5 g1f3 d7d6 d2d4 c8g4 d4e5 g4f3 d1f3 d6e5 f1c4 g8f6 f3b3 d8e7 b1c3 c7c6 c1g5 b7b5 c3b5 c6b5 c4b5 "
         "b8d7 e1c1 a8d8 d1d7 d8d7 h1d1 e7e6 b5d7 f6d7 b3b8 d7b8 d1d8").split()
# en passant, an under-promotion with capture, short castling for both sides
SAN_B = "e4 a6 e5 d5 exd6 a5 dxc7 a4 cxb8=N Nf6 Nf3 e6 Be2 Be7 O-O O-O Nc6 bxc6".split()
UCI_B = "e2e4 a7a6 e4e5 d7d5 e5d6 a6a5 d6c7 a5a4 c7b8n g8f6 g1f3 e7e6 f1e2 f8e7 e1g1 e8g8 b8c6 b7c6".split()


def oracle_replay(uci_moves):
    pos = chesspos.Position()
    hist = [pos.copy()]
    for u in uci_moves:
        (move,) = [m for m in pos.legal_moves() if chesspos.uci(m) == u]
        pos.push(move)
        hist.append(pos.copy())
    return hist


@pytest.mark.parametrize("san,uci", [(SAN_A, UCI_A), (SAN_B, UCI_B)])
def test_game_replay_matches_oracle(lib, san, uci):
    from chessrl_b200 import positions
    hist = oracle_replay(uci)
    for moves in (san, uci):
        got = positions.game_records(moves, legal=True, fens=True)
        assert got["fens"] == [p.fen() for p in hist]
        for i, pos in enumerate(hist):
            recent = hist[max(0, i - 7):i + 1][::-1]
            want = chesspos.pack_planes104(chesspos.planes112(recent, rule50=True)[None])[0]
            np.testing.assert_array_equal(got["packed"][i].numpy(), want)
            view = pos.mirror() if pos.turn == chesspos.BLACK else pos
            np.testing.assert_array_equal(got["legal1858"][i].numpy(), chesspos.legal_bits(view, 1858))
            assert int(got["black"][i]) == pos.turn
    part = positions.game_records(san, first_ply=8, count=3)
    assert torch.equal(part["packed"], positions.game_records(uci)["packed"][8:11])
    for bad in (["e4", "Ke2"], ["e4", "e5", "Nc3", "Nc6", "Ne2", "d6", "Nc3x"], ["Nf3", "Nf6", "N3"], ["e9"]):
        with pytest.raises(ValueError):
            positions.game_records(bad)
    with pytest.raises(ValueError):
        positions.game_records(["Nge2"])                       # e2 holds a pawn: no legal move matches
    assert positions.game_records(["Ngf3"])["packed"].shape == (2, 840)   # redundant disambiguation still selects one move


class StandInEngine:
    """Answers with rows that encode the record they were computed from, so that the test can follow every
    position through pooling and splitting."""

    def __init__(self):
        self.calls = []

    def forward(self, packed, **kw):
        assert kw["layout"] == "packed104" and kw["host"] and kw["legal_mask"] == "records" and kw["rl_vocab"]
        self.calls.append(int(packed.shape[0]))
        key = packed.to(torch.int64).sum(dim=1) % 1009
        rows = torch.zeros(packed.shape[0], 1929, dtype=torch.float16)
        rows[:, 0] = key.to(torch.float16) / 1024
        rows[:, 1] = kw["black_rows"].to(torch.float16)
        return {"policy": rows}


def expected_rows(pre, post):
    from chessrl_b200 import positions
    g = positions.game_records(pre + post, first_ply=len(pre), count=len(post), rule50_plane=False)   # the server's default
    assert int(g["packed"][:, 837].max()) == 0                 # plane 109 stays empty, as in the reference server's input
    rows = np.zeros((len(post), 1929), dtype=np.float16)
    rows[:, 0] = ((g["packed"].to(torch.int64).sum(dim=1) % 1009).to(torch.float16) / 1024).numpy()
    rows[:, 1] = g["black"].numpy()
    return rows


def test_server_protocol_pooling_and_rejections(lib):
    from chessrl_b200 import server
    eng = StandInEngine()
    srv = server.PolicyServer(eng, port=0, max_positions=64, linger_ms=300.0).start()
    try:
        reqs = [[(SAN_A[:8], SAN_A[8:20]), (UCI_B[:9], UCI_B[9:])], [(UCI_A[:7], UCI_A[7:10])]]
        answers = [None, None]

        def ask(i):
            answers[i] = server.query(srv.address, reqs[i])

        threads = [threading.Thread(target=ask, args=(i,)) for i in range(2)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=30)
        for req, ans in zip(reqs, answers):
            assert isinstance(ans, list) and len(ans) == len(req)
            for (pre, post), rows in zip(req, ans):
                assert rows.dtype == np.float16 and rows.shape == (len(post), 1929)
                np.testing.assert_array_equal(rows, expected_rows(pre, post))
        assert sum(eng.calls) == 12 + 9 + 3 and len(eng.calls) == 1          # both connections pooled into one engine call
        # requests the reference would fail on get the empty answer, and the connection stays usable
        assert server.query(srv.address, [(SAN_A[:3], SAN_A[3:6])]) is None  # fewer than 7 moves of history
        assert server.query(srv.address, [(SAN_A[:8], ["Qh5"])]) is None      # not a legal move there
        ok = server.query(srv.address, [(SAN_A[:8], SAN_A[8:9])])
        np.testing.assert_array_equal(ok[0], expected_rows(SAN_A[:8], SAN_A[8:9]))
    finally:
        srv.close()
    # a length prefix beyond the limit ends the connection instead of reserving the memory
    import socket as _socket
    import struct as _struct
    a, b = _socket.socketpair()
    a.sendall(_struct.pack(">Q", 1 << 60))
    assert server.recv_message(b) is None
    a.close()
    b.close()
    # a pickle that names any global is refused before anything is called
    for evil in (pickle.dumps(os.getcwd), pickle.dumps([[["e4"], [print]]])):
        with pytest.raises(pickle.UnpicklingError):
            server.decode_request(evil)
    with pytest.raises(ValueError):
        server.decode_request(pickle.dumps({"a": 1}))
