"""Policy server speaking the wire protocol of the reference's Leela/server.py (lines 113-166; client side
Leela/client_final_final.py:91-135): every message is an 8-byte big-endian length followed by a pickle.

Request  : a list of [pre_moves, post_moves] pairs (lists of SAN or UCI strings, len(pre_moves) >= 7 as the
           reference asserts in pgn_to_input_data_decoder.py:16). For each pair the positions after
           pre_moves + post_moves[:j], j = 0 .. len(post_moves)-1, are evaluated.
Response : a list with one float16 array [len(post_moves), 1929] per pair - softmax(mask + logits) over the
           1858 Leela moves scattered into the 1929-entry vocabulary, Black rows rank-mirrored
           (server.py:54-62: batched_inference, softmax, map_leela_to_rl). An empty payload (length 0) answers a
           request that could not be evaluated, as the reference does.

What differs from the reference loop: requests of all connections are pooled by one batching thread into engine
calls of up to `max_positions` positions (the reference serves one client at a time, 2048 rows per model call);
positions travel to the GPU as 840-byte packed records, the legal-move masks are generated there, and the pickle
reader only accepts lists, tuples and strings (a pickle is code; the reference loads whatever arrives).
"""
import io
import pickle
import queue
import socket
import struct
import threading
import time

import numpy as np
import torch

from . import positions

HEADER = struct.Struct(">Q")


class _ListsOfStrings(pickle.Unpickler):
    """Unpickler for the request format only: no global may be resolved, so no callable can be reached."""

    def find_class(self, module, name):
        raise pickle.UnpicklingError(f"request tried to load {module}.{name}")


def decode_request(payload):
    req = _ListsOfStrings(io.BytesIO(payload)).load()
    if not isinstance(req, (list, tuple)):
        raise ValueError("request is not a list")
    out = []
    for item in req:
        if not isinstance(item, (list, tuple)) or len(item) != 2:
            raise ValueError("request items are [pre_moves, post_moves]")
        pre, post = item
        if not all(isinstance(m, str) for m in list(pre) + list(post)):
            raise ValueError("moves are strings")
        out.append((list(pre), list(post)))
    return out


def recv_exact(sock, n):
    buf = bytearray(n)
    view = memoryview(buf)
    got = 0
    while got < n:
        k = sock.recv_into(view[got:], n - got)
        if k == 0:
            return None
        got += k
    return bytes(buf)


def send_message(sock, payload):
    sock.sendall(HEADER.pack(len(payload)) + payload)


MAX_MESSAGE_BYTES = 256 << 20      # a length beyond this is treated as a broken peer, not as memory to reserve


def recv_message(sock):
    head = recv_exact(sock, HEADER.size)
    if head is None:
        return None
    (n,) = HEADER.unpack(head)
    if n > MAX_MESSAGE_BYTES:
        return None
    return recv_exact(sock, n) if n else b""


def records_for(pairs, rule50_plane=False):
    """Packed records, Black flags and per-pair position counts of a decoded request. rule50_plane=False leaves
    plane 109 empty, as the reference server's input does (Leela/ustotheirs.py:13-17 appends a blank plane there);
    True writes halfmove/100 for networks trained on lc0 records."""
    packed, black, counts = [], [], []
    for pre, post in pairs:
        if len(pre) + 1 < 8:
            raise ValueError("at least 7 moves must precede the first evaluated position")
        k = len(post)
        counts.append(k)
        if k == 0:
            continue
        g = positions.game_records(pre + post, first_ply=len(pre), count=k, rule50_plane=rule50_plane)
        packed.append(g["packed"])
        black.append(g["black"])
    if not packed:
        return torch.empty(0, 840, dtype=torch.uint8), torch.empty(0, dtype=torch.uint8), counts
    return torch.cat(packed), torch.cat(black), counts


class PolicyServer:
    """`engine`: a chessrl_b200.Engine with the 112-plane gather head (or any object with the same
    forward(packed, layout=..., host=True, ...) -> {"policy": [B,1929] f16 tensor} call)."""

    def __init__(self, engine, host="127.0.0.1", port=65432, max_positions=2048, linger_ms=2.0, rule50_plane=False):
        self.engine = engine
        self.max_positions = max_positions
        self.linger = linger_ms * 1e-3
        self.rule50_plane = rule50_plane
        self._jobs = queue.Queue()
        self._stop = threading.Event()
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((host, port))
        self._sock.listen()
        self._sock.settimeout(0.2)
        self.address = self._sock.getsockname()
        self.batches = []            # positions per engine call, for tests and monitoring
        self._threads = [threading.Thread(target=self._accept_loop, daemon=True),
                         threading.Thread(target=self._batch_loop, daemon=True)]

    def start(self):
        for t in self._threads:
            t.start()
        return self

    def close(self):
        self._stop.set()
        for t in self._threads:
            t.join(timeout=5)
        self._sock.close()

    # ---- connections -----------------------------------------------------------------------------
    def _accept_loop(self):
        while not self._stop.is_set():
            try:
                conn, _ = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn):
        with conn:
            conn.settimeout(None)
            while not self._stop.is_set():
                payload = recv_message(conn)
                if payload is None:
                    return
                try:
                    packed, black, counts = records_for(decode_request(payload), self.rule50_plane)
                except Exception:
                    send_message(conn, b"")            # the reference answers a failed prediction with length 0
                    continue
                done = threading.Event()
                job = {"packed": packed, "black": black, "done": done, "rows": None}
                self._jobs.put(job)
                done.wait()
                if job["rows"] is None:
                    send_message(conn, b"")
                    continue
                rows, out, at = job["rows"], [], 0
                for k in counts:
                    out.append(rows[at:at + k])
                    at += k
                send_message(conn, pickle.dumps(out))

    # ---- batching --------------------------------------------------------------------------------
    def _batch_loop(self):
        while not self._stop.is_set():
            try:
                first = self._jobs.get(timeout=0.1)
            except queue.Empty:
                continue
            jobs, n = [first], first["packed"].shape[0]
            deadline = time.monotonic() + self.linger
            while n < self.max_positions:
                left = deadline - time.monotonic()
                if left <= 0:
                    break
                try:
                    j = self._jobs.get(timeout=left)
                except queue.Empty:
                    break
                jobs.append(j)
                n += j["packed"].shape[0]
            try:
                rows = self._evaluate(torch.cat([j["packed"] for j in jobs]), torch.cat([j["black"] for j in jobs]))
                at = 0
                for j in jobs:
                    k = j["packed"].shape[0]
                    j["rows"] = rows[at:at + k]
                    at += k
            except Exception:
                pass                                     # rows stay None: every waiting client gets the empty answer
            for j in jobs:
                j["done"].set()

    def _evaluate(self, packed, black):
        self.batches.append(int(packed.shape[0]))
        if packed.shape[0] == 0:
            return np.zeros((0, 1929), dtype=np.float16)
        out = self.engine.forward(packed, layout="packed104", host=True, legal_mask="records", policy_softmax=True,
                                  policy_dtype=torch.float16, rl_vocab=True, black_rows=black, wdl=False)
        return out["policy"].numpy()


def query(address, pairs, timeout=60.0):
    """Client side of the protocol (Leela/client_final_final.py:91-135): one request, one response."""
    with socket.create_connection(address, timeout=timeout) as s:
        send_message(s, pickle.dumps([[list(a), list(b)] for a, b in pairs]))
        payload = recv_message(s)
    if not payload:
        return None
    return pickle.loads(payload)
