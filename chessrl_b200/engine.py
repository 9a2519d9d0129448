"""Python face of the C ABI: an `Engine` owns one `crl_handle` on one GPU and moves torch tensors in
and out by raw pointer. torch is used for device memory and streams only; all arithmetic happens in
libchessrl_b200.so."""
import ctypes
from dataclasses import dataclass, asdict

import torch

from . import _lib as L


@dataclass
class EngineConfig:
    """Mirror of `crl_config` (include/chessrl_b200.h)."""
    planes: int = 112
    d_model: int = 512
    n_layers: int = 10
    n_heads: int = 8
    d_ff: int = 736
    ln_mode: int = L.LN_POST
    act: int = L.ACT_GELU
    ffn_act_pos: int = L.FFN_ACT_END
    bias_mode: int = L.BIAS_RELPOS
    policy_mode: int = L.POLICY_DENSE4096
    value_mode: int = L.VALUE_WDL_Q
    dtype: int = L.DTYPE_F16
    smolgen_compress: int = 32
    smolgen_hidden: int = 256
    smolgen_gen: int = 256
    chunk: int = 0
    pos_embed: int = 0
    lm_vocab: int = 0
    fuse_layernorm: int = L.FUSE_LN_AUTO
    precision: int = 0

    @staticmethod
    def reference_value_q(n_layers=10, d_model=512, d_ff=736, n_heads=8, **kw):
        """`BT4(num_layers, d_model, d_ff, num_heads)` of new_paradigm/value_q.py:122 (112 planes)."""
        return EngineConfig(112, d_model, n_layers, n_heads, d_ff, **kw)

    @staticmethod
    def reference_value(n_layers=10, d_model=512, d_ff=736, n_heads=8, **kw):
        """`BT4` of new_paradigm/value.py:122 (19 planes, WDL head)."""
        return EngineConfig(19, d_model, n_layers, n_heads, d_ff, value_mode=L.VALUE_WDL, **kw)

    @staticmethod
    def baseline(n_layers, d_model, d_ff, n_heads, smolgen=True, value_only=False, **kw):
        """Network of the target specification: post-LN, Mish between ff1 and ff2, smolgen bias, gather
        policy over the 1858 Leela moves, WDL head."""
        return EngineConfig(112, d_model, n_layers, n_heads, d_ff, L.LN_POST, L.ACT_MISH, L.FFN_ACT_MID,
                            L.BIAS_SMOLGEN if smolgen else L.BIAS_NONE,
                            L.POLICY_NONE if value_only else L.POLICY_GATHER1858, L.VALUE_WDL, **kw)

    @staticmethod
    def reference_gpt(n_layer=6, n_head=12, n_embd=768, vocab_size=1929, **kw):
        """Board-only path of `GPT(GPTConfig)` (model_bis.py:127-156, 358-370): 19 planes, pre-LN causal
        blocks, GELU MLP 4x, final LayerNorm, last-token LM head."""
        return EngineConfig(19, n_embd, n_layer, n_head, 4 * n_embd, L.LN_PRE, L.ACT_GELU, L.FFN_ACT_MID, L.BIAS_CAUSAL,
                            L.POLICY_LM_HEAD, L.VALUE_NONE, pos_embed=1, lm_vocab=vocab_size, **kw)

    def to_c(self):
        return L.Config(**asdict(self))


_LAYOUT_OF = {
    ("nhwc", torch.float32): L.LAYOUT_NHWC_F32, ("nhwc", torch.float16): L.LAYOUT_NHWC_F16,
    ("nchw", torch.float16): L.LAYOUT_NCHW_F16, ("nchw", torch.float32): L.LAYOUT_NCHW_F32,
    ("packed104", torch.uint8): L.LAYOUT_PACKED104,
}


def check_rows(name, t, dev, rows, dtypes):
    """Raise ValueError unless tensor `t` lives on the device type of `dev`, has `rows` rows and one of `dtypes`.
    The library receives raw pointers and cannot see any of this: a host pointer or a short buffer handed to a
    kernel would be an illegal address on the GPU."""
    if not (hasattr(t, "device") and hasattr(t, "dtype") and hasattr(t, "shape")):
        raise ValueError(f"{name} must be a tensor")
    if t.device.type != dev.type or (dev.type == "cuda" and dev.index is not None and t.device.index != dev.index):
        raise ValueError(f"{name} must live on {dev}, got {t.device}")
    if t.dtype not in dtypes:
        raise ValueError(f"{name} must have dtype {' or '.join(str(d) for d in dtypes)}, got {t.dtype}")
    if t.dim() < 1 or t.shape[0] != rows:
        raise ValueError(f"{name} must have {rows} rows, got shape {tuple(t.shape)}")


def check_forward_inputs(planes, dev, batch, n_moves, legal_mask=None, mask_mode=None, black_rows=None, uniforms=None,
                         rl_vocab=False):
    """Every device / shape / dtype rule of Engine.forward's tensor arguments, checked before any pointer
    reaches the library (no kernel has been launched when this raises)."""
    if planes.device.type != dev.type or (dev.type == "cuda" and dev.index is not None and planes.device.index != dev.index):
        raise ValueError(f"planes must live on {dev}")
    if legal_mask is not None and not isinstance(legal_mask, str):
        check_rows("legal_mask", legal_mask, dev, batch, (torch.uint8, torch.float32))
        if legal_mask.dim() != 2:
            raise ValueError("legal_mask must be [B, ceil(V/8)] uint8 or [B, V] float32")
        bits = legal_mask.dtype == torch.uint8 if mask_mode is None else mask_mode == L.MASK_BITS
        if bits != (legal_mask.dtype == torch.uint8):
            raise ValueError("mask_mode does not match the dtype of legal_mask (bitset: uint8, additive: float32)")
        need = (n_moves + 7) // 8 if bits else n_moves
        if legal_mask.shape[1] < need:
            raise ValueError(f"legal_mask rows hold {legal_mask.shape[1]} entries, the move list needs {need}")
    if black_rows is not None and rl_vocab:
        check_rows("black_rows", black_rows, dev, batch, (torch.uint8,))
        if black_rows.numel() != batch:
            raise ValueError("black_rows must be [B]")
    if uniforms is not None:
        check_rows("uniforms", uniforms, dev, batch, (torch.float32,))
        if uniforms.numel() != batch:
            raise ValueError(f"uniforms must be [B] on {dev}")


class Engine:
    def __init__(self, cfg: EngineConfig, device=0):
        self.lib = L.load()
        self.cfg = cfg
        self.device = torch.device("cuda", device) if not isinstance(device, torch.device) else device
        self._h = ctypes.c_void_p()
        c = cfg.to_c()
        rc = self.lib.crl_create(ctypes.byref(c), self.device.index or 0, ctypes.byref(self._h))
        if rc != 0:
            raise L.CrlError(rc, "crl_create")
        self._ws = None
        self.n_moves = self.lib.crl_num_moves(self._h)

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            self.lib.crl_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what):
        if rc != 0:
            raise L.CrlError(rc, f"{what}: {self.lib.crl_error_detail(self._h).decode()}")

    # ---- weights ---------------------------------------------------------------------------------
    def required_keys(self):
        n = self.lib.crl_num_required_keys(self._h)
        return [self.lib.crl_required_key(self._h, i).decode() for i in range(n)]

    def load_state_dict(self, sd):
        """Push every key the configuration needs (reference names) and repack. Extra keys in `sd`
        are ignored, a missing one raises (CRL_ERR_MISSING_WEIGHT names it)."""
        for k in self.required_keys():
            if k not in sd:
                raise L.CrlError(-4, k)
            t = sd[k].detach().to(dtype=torch.float32).contiguous()
            if t.is_cuda:
                torch.cuda.synchronize(t.device)
            self._check(self.lib.crl_set_weight(self._h, k.encode(), t.data_ptr(), t.numel()), f"set_weight {k}")
        self._check(self.lib.crl_finalize(self._h), "finalize")

    # ---- scratch ---------------------------------------------------------------------------------
    def workspace(self, batch):
        need = self.lib.crl_workspace_bytes(self._h, batch)
        if self._ws is None or self._ws.numel() < need:
            self._ws = None
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._ws

    @staticmethod
    def _layout(planes, layout):
        key = (layout, planes.dtype)
        if key not in _LAYOUT_OF:
            raise ValueError(f"unsupported planes layout/dtype {key}")
        return _LAYOUT_OF[key]

    def _batch_of(self, planes, layout):
        p = self.cfg.planes
        if layout == "packed104":
            if planes.dim() != 2 or planes.shape[1] != L.PACKED104_BYTES:
                raise ValueError(f"packed planes are [B, {L.PACKED104_BYTES}] uint8")
            return planes.shape[0]
        if planes.numel() % (64 * p) != 0:
            raise ValueError("planes tensor is not a whole number of positions")
        if layout == "nhwc" and planes.shape[-1] != p:
            raise ValueError(f"expected {p} planes in the last dimension, got {planes.shape[-1]}")
        return planes.numel() // (64 * p)

    def calibrate(self, planes, layout="nhwc"):
        """FP8 engines: fix the per-tensor activation scales from this batch (device tensor)."""
        planes = planes.contiguous()
        b = self._batch_of(planes, layout)
        ws = self.workspace(b)
        s = torch.cuda.current_stream(self.device).cuda_stream
        self._check(self.lib.crl_calibrate(self._h, planes.data_ptr(), self._layout(planes, layout), b, ws.data_ptr(),
                                           ws.numel(), s), "calibrate")

    # ---- forward ---------------------------------------------------------------------------------
    def forward(self, planes, layout="nhwc", legal_mask=None, mask_mode=None, policy=True, wdl=True, q=False,
                policy_softmax=False, wdl_softmax=True, policy_dtype=torch.float32, host=False, rl_vocab=False,
                black_rows=None, moves=False, temperature=0.0, uniforms=None):
        """planes: [..., 8, 8, P] ("nhwc"), [B, P, 8, 8] ("nchw") or [B, 840] uint8 bit-packed records
        ("packed104", see positions.pack_planes104), on the engine's GPU (or on the host
        with host=True, which times like a user call: copies in, run, copies out, synchronise).
        legal_mask: uint8 bitset [B, ceil(V/8)] (bit m of row b: move m legal), float32 additive [B, V], or the
        string "records" (packed104 input, gather head): the legal moves are generated on the GPU.
        rl_vocab=True (gather head): rows of 1929 in the reference's own vocabulary, Black rows (uint8 flags in
        `black_rows`) rank-mirrored, like `map_leela_to_rl` after the server's softmax.
        moves=True: the move per position is chosen on the GPU (model_bis.py:385-394): arg-max for temperature 0
        or without `uniforms`, else the inverse-CDF draw of softmax(logits / temperature) for the caller's
        uniform numbers [B] in [0,1); `move` [B] int32 indexes the policy row. With policy=False only the
        indices come back (4 bytes per position instead of the row).
        Returns a dict with `policy` [B, V], `wdl` [B, 3], `q` [B], `move` [B] as requested and available."""
        planes = planes.contiguous()
        b = self._batch_of(planes, layout)
        dev = torch.device("cpu") if host else self.device
        if black_rows is not None:
            black_rows = black_rows.to(torch.uint8).contiguous()
        if uniforms is not None:
            uniforms = uniforms.to(torch.float32).contiguous()
        check_forward_inputs(planes, dev, b, self.n_moves, legal_mask, mask_mode, black_rows, uniforms, rl_vocab)
        io = L.IO()
        io.planes = planes.data_ptr()
        io.layout = self._layout(planes, layout)
        io.batch = b
        out = {}
        if isinstance(legal_mask, str):
            if legal_mask != "records":
                raise ValueError('legal_mask is a tensor or the string "records"')
            io.mask_mode = L.MASK_FROM_RECORDS      # legal moves generated on the GPU from the packed records
        elif legal_mask is not None:
            legal_mask = legal_mask.contiguous()
            if mask_mode is None:
                mask_mode = L.MASK_BITS if legal_mask.dtype == torch.uint8 else L.MASK_ADDITIVE
            io.legal_mask = legal_mask.data_ptr()
            io.mask_mode = mask_mode
            io.mask_stride = legal_mask.shape[-1]
        want_policy = policy and self.n_moves > 0
        want_moves = moves and self.n_moves > 0
        kw = dict(device=dev, pin_memory=True) if host else dict(device=dev)
        if want_policy or want_moves:
            width = 1929 if rl_vocab else self.n_moves
            io.policy_softmax = int(policy_softmax)
            if want_policy or not host:      # the device entry point reads the moves from caller-owned rows
                rows = torch.empty(b, width, dtype=policy_dtype, **kw)
                io.policy_out = rows.data_ptr()
                io.policy_dtype = L.OUT_F32 if policy_dtype == torch.float32 else L.OUT_F16
                io.policy_stride = width
                if want_policy:
                    out["policy"] = rows
            if want_moves:
                out["move"] = torch.empty(b, dtype=torch.int32, **kw)
                io.move_out = out["move"].data_ptr()
                io.move_temperature = float(temperature)
                if uniforms is not None:
                    io.move_uniform = uniforms.data_ptr()
            if rl_vocab:
                io.policy_vocab = L.VOCAB_RL1929
                if black_rows is not None:
                    io.black_rows = black_rows.data_ptr()
        if wdl and self.cfg.value_mode != L.VALUE_NONE:
            out["wdl"] = torch.empty(b, 3, dtype=torch.float32, **kw)
            io.wdl_out = out["wdl"].data_ptr()
            io.wdl_softmax = int(wdl_softmax)
        if q and self.cfg.value_mode == L.VALUE_WDL_Q:
            out["q"] = torch.empty(b, dtype=torch.float32, **kw)
            io.q_out = out["q"].data_ptr()
        io.stream = torch.cuda.current_stream(self.device).cuda_stream
        if host:
            self._check(self.lib.crl_forward_host(self._h, ctypes.byref(io)), "forward_host")
        else:
            ws = self.workspace(b)
            io.workspace = ws.data_ptr()
            io.workspace_bytes = ws.numel()
            self._check(self.lib.crl_forward(self._h, ctypes.byref(io)), "forward")
        return out

    def legal_masks(self, packed):
        """[B, 840] uint8 packed records on the engine's GPU -> [B, 233] uint8 legal-move bitsets over the 1858-move
        list in the mover's view, generated on the GPU (the rows `positions.playout_positions` calls legal1858)."""
        packed = packed.contiguous()
        if packed.dim() != 2 or packed.shape[1] != L.PACKED104_BYTES or packed.dtype != torch.uint8 or packed.device.type != "cuda":
            raise ValueError("packed records are [B, 840] uint8 on the GPU")
        out = torch.empty(packed.shape[0], 233, dtype=torch.uint8, device=packed.device)
        s = torch.cuda.current_stream(self.device).cuda_stream
        self._check(self.lib.crl_legal_masks_packed104(self._h, packed.data_ptr(), packed.shape[0], out.data_ptr(), 233, s),
                    "legal_masks")
        return out

    def last_status(self):
        st = ctypes.c_int(0)
        rc = self.lib.crl_last_status(self._h, ctypes.byref(st))
        return rc, st.value

    def last_launch_count(self):
        return int(self.lib.crl_last_launch_count(self._h))

    def profile(self, enable=True):
        """Turn per-kernel event timing on (clearing earlier records) or off."""
        self._check(self.lib.crl_profile(self._h, int(enable)), "profile")

    def profile_read(self):
        """{category: dict(ms, flops, bytes, launches)} summed over the launches recorded since profile(True)."""
        out = {}
        for cat, name in enumerate(("gemm", "attention", "layernorm", "policy")):
            ms, fl, by, n = ctypes.c_double(), ctypes.c_double(), ctypes.c_double(), ctypes.c_int64()
            self._check(self.lib.crl_profile_read(self._h, cat, ctypes.byref(ms), ctypes.byref(fl), ctypes.byref(by),
                                                  ctypes.byref(n)), "profile_read")
            out[name] = dict(ms=ms.value, flops=fl.value, bytes=by.value, launches=n.value)
        return out

    def profile_entries(self):
        """Every recorded launch in order: dict(cat, ms, flops, bytes, m, n, k, kind)."""
        out, i = [], 0
        while True:
            cat, ms, fl, by = ctypes.c_int(), ctypes.c_double(), ctypes.c_double(), ctypes.c_double()
            mnk = (ctypes.c_int * 4)()
            rc = self.lib.crl_profile_entry(self._h, i, ctypes.byref(cat), ctypes.byref(ms), ctypes.byref(fl),
                                            ctypes.byref(by), ctypes.byref(mnk))
            if rc != 0:
                return out
            out.append(dict(cat=cat.value, ms=ms.value, flops=fl.value, bytes=by.value, m=mnk[0], n=mnk[1], k=mnk[2],
                            kind=mnk[3]))
            i += 1
