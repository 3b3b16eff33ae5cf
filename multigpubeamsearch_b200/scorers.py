"""Device scorers that plug into BeamEngine.set_scorer.

The reference's scorers.py wraps torch modules (MLPActionScorer 120->1024->256->24, scorers.py:21-53) and its C++
engine runs them through InferenceBackend::forward.  Here the scorer is a value network on child states, evaluated
by hand-written tcgen05 GEMM kernels inside libmgbs_b200.so; this module only prepares weights and work buffers
(torch tensors) and hands the native object to the engine.
"""

from __future__ import annotations

import ctypes as C
from typing import Any, Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from . import _lib
from .records import unpack_payload  # noqa: F401  (re-exported for callers of the engine)

MAX_MODELS = 4


class MgbsMlpConfig(C.Structure):
    _fields_ = [
        ("state_len", C.c_int32), ("state_stride", C.c_int32), ("num_values", C.c_int32), ("hidden", C.c_int32),
        ("num_models", C.c_int32), ("k1_pad", C.c_int32), ("max_rows", C.c_int64), ("score_offset", C.c_float),
        ("b3", C.c_float * MAX_MODELS),
        ("x", C.c_void_p), ("h1", C.c_void_p), ("q", C.c_void_p), ("err", C.c_void_p),
        ("w1", C.c_void_p * MAX_MODELS), ("b1", C.c_void_p * MAX_MODELS), ("w2", C.c_void_p * MAX_MODELS),
        ("b2", C.c_void_p * MAX_MODELS), ("w3", C.c_void_p * MAX_MODELS),
        ("s1", C.c_void_p * MAX_MODELS), ("s2", C.c_void_p * MAX_MODELS),
        ("dtype", C.c_int32), ("act_inv_scale", C.c_float),
        ("h1q", C.c_void_p), ("sf_h1", C.c_void_p), ("sf_w2", C.c_void_p * MAX_MODELS),
        ("act4_inv_global", C.c_float), ("pad0", C.c_int32),
    ]


E2M1_MIDPOINTS = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])


def e2m1_codes(x: np.ndarray) -> np.ndarray:
    """4-bit E2M1 codes (sign in bit 3) of x rounded to the nearest representable value, ties to the even code."""
    a = np.abs(np.asarray(x, dtype=np.float64))
    code = np.searchsorted(E2M1_MIDPOINTS, a, side="left")
    tie = (code < 7) & (a == E2M1_MIDPOINTS[np.minimum(code, 6)])
    code = np.where(tie & (code % 2 == 1), code + 1, code).astype(np.uint8)
    return code | (np.signbit(x).astype(np.uint8) << 3)


def nvfp4_quantize_weights(w: np.ndarray):
    """NVFP4 form of a weight matrix [N, K] (N a multiple of 256, K of 256) for the block-scaled tensor-core path:
    (packed E2M1 bytes [N, K/2] with even K in the low nibble, block factors as bytes in the kernel's tile order
    [N/256][K/256][2 groups of 128 rows][4 steps][512], tensor scale)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    if n % 256 or k % 256:
        raise RuntimeError("NVFP4 weights need dimensions that are multiples of 256")
    tscale = np.float32(max(float(np.abs(w).max()), 1e-30) / (6.0 * 448.0))
    blocks = w.reshape(n, k // 16, 16)
    amax = np.abs(blocks).max(axis=2)
    sf8 = torch.from_numpy((amax / np.float32(6.0) / tscale).astype(np.float32)).to(torch.float8_e4m3fn)
    sf = sf8.to(torch.float32).numpy()
    step = (sf * tscale)[:, :, None]
    scaled = np.where(step > 0, blocks / np.where(step > 0, step, 1.0), 0.0)
    codes = e2m1_codes(scaled).reshape(n, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    # factors: row r of group g (128 rows) of chunk c (256 rows), K-block kb, step st, block j ->
    # tile (c, kb, g, st) byte (r % 32) * 16 + (r // 32) * 4 + j
    # the two 128-row groups of a 256-row chunk sit side by side, so one K-block of a 256-column tile is one 4 KB run
    sfb = sf8.view(torch.uint8).numpy().reshape(n // 256, 2, 4, 32, k // 256, 4, 4)  # [c, g, r1, r0, kb, st, j]
    sfb = np.ascontiguousarray(sfb.transpose(0, 4, 1, 5, 3, 2, 6))                    # [c, kb, g, st, r0, r1, j]
    return np.ascontiguousarray(packed), sfb.reshape(-1).copy(), float(tscale)


def onehot_columns(state_len: int, num_values: int) -> int:
    """Width of the one-hot operand in the column order of the layer-1 kernels: column = value * P + position with
    P = state_len rounded up to 8 (eight adjacent columns = one byte-compare of the state row)."""
    return num_values * ((state_len + 7) // 8 * 8)


def onehot_relayout(w1: np.ndarray, state_len: int, num_values: int, k1_pad: int) -> np.ndarray:
    """[H, state_len * num_values] with column position * V + value (the layout of Linear weights on a flattened
    one-hot, scorers.py:21-36) -> [H, k1_pad] float32 in the kernels' column order, zero padded."""
    w1 = np.asarray(w1, dtype=np.float32)
    h = w1.shape[0]
    p = (state_len + 7) // 8 * 8
    out = np.zeros((h, k1_pad), dtype=np.float32)
    src = w1.reshape(h, state_len, num_values)
    out[:, : num_values * p].reshape(h, num_values, p)[:, :, :state_len] = src.transpose(0, 2, 1)
    return out


_E2M1_VALUES = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)


def nvfp4_round_weights(w: np.ndarray) -> np.ndarray:
    """A weight matrix [N, K] (K a multiple of 16) rounded to the NVFP4 grid and returned as float32: per block of 16
    consecutive K elements one E4M3 factor e4m3(blockmax / 6 / tensor scale), elements E2M1, tensor scale
    max|w| / (6 * 448).  The values the block-scaled tensor-core path would multiply with (nvfp4_quantize_weights
    packs the same numbers)."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    n, k = w.shape
    if k % 16:
        raise RuntimeError("NVFP4 blocks need K to be a multiple of 16")
    tscale = np.float32(max(float(np.abs(w).max()), 1e-30) / (6.0 * 448.0))
    blocks = w.reshape(n, k // 16, 16)
    amax = np.abs(blocks).max(axis=2)
    sf = torch.from_numpy((amax / np.float32(6.0) / tscale).astype(np.float32)).to(torch.float8_e4m3fn).to(torch.float32).numpy()
    step = (sf * tscale)[:, :, None]
    scaled = np.where(step > 0, blocks / np.where(step > 0, step, 1.0), 0.0)
    codes = e2m1_codes(scaled)
    vals = np.where(codes & 8, -1.0, 1.0).astype(np.float32) * _E2M1_VALUES[codes & 7]
    return (vals * step).reshape(n, k).astype(np.float32)


class MgbsMlpNoAllocArgs(C.Structure):
    _fields_ = [
        ("state_len", C.c_int32), ("state_stride", C.c_int32), ("num_values", C.c_int32), ("hidden", C.c_int32),
        ("score_offset", C.c_float), ("b3", C.c_float),
        ("w1", C.c_void_p), ("b1", C.c_void_p), ("w2", C.c_void_p), ("b2", C.c_void_p), ("w3", C.c_void_p),
    ]


NOALLOC_MAX_ROWS = 4096

_SIGS = {
    "mgbs_mlp_score_noalloc": (C.c_int, [C.POINTER(MgbsMlpNoAllocArgs), C.c_void_p, C.c_int32, C.c_void_p,
                                         C.POINTER(C.c_int32), C.c_void_p]),
    "mgbs_sizeof_mlp_config": (C.c_int, []),
    "mgbs_mlp_create": (C.c_int, [C.POINTER(MgbsMlpConfig), C.POINTER(C.c_void_p)]),
    "mgbs_mlp_destroy": (C.c_int, [C.c_void_p]),
    "mgbs_mlp_profile": (C.c_int, [C.c_void_p, C.c_int32]),
    "mgbs_mlp_set_l1_mode": (C.c_int, [C.c_void_p, C.c_int32]),
    "mgbs_mlp_set_head_mode": (C.c_int, [C.c_void_p, C.c_int32]),
    "mgbs_mlp_set_l1_variant": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32]),
    "mgbs_mlp_profile_read": (C.c_int, [C.c_void_p, C.POINTER(C.c_float)]),
    "mgbs_mlp_enqueue": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}
_lib.SIGNATURES.update(_SIGS)


class MLPValueScorer:
    """Ensemble of value MLPs one-hot(n*V) -> hidden -> hidden -> 1 (ReLU); bf16 or FP8 (E4M3) operands, fp32
    accumulation.

    ``dtype="fp8"``: weights are quantised to E4M3 with one scale per output channel (max-abs / 448); first-layer
    activations are stored as E4M3 with one per-tensor scale taken from a safe bound on their maximum
    (sum over positions of the largest first-layer weight of that position, plus bias).

    ``weights``: one dict or a list of dicts with float32 arrays w1 [H, n*V], b1 [H], w2 [H, H], b2 [H], w3 [H], b3.
    ``score_offset``: subtracted from the network output before it becomes the integer key
    ``uint32(clamp(q - offset, 0, 300) * 256 + 0.5)``; choose it so that outputs land inside [0, 300].
    """

    def __init__(self, weights: Union[Dict[str, np.ndarray], Sequence[Dict[str, np.ndarray]]], state_len: int,
                 state_stride: int, num_values: int, max_rows: int, score_offset: float = -150.0,
                 device: Union[str, torch.device, None] = None, dtype: str = "bf16"):
        self.lib = _lib.load()
        for name, (res, args) in _SIGS.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args
        if self.lib.mgbs_sizeof_mlp_config() != C.sizeof(MgbsMlpConfig):
            raise RuntimeError("structure layout mismatch between scorers.py and libmgbs_b200.so")
        if isinstance(weights, dict):
            weights = [weights]
        if not 1 <= len(weights) <= MAX_MODELS:
            raise RuntimeError(f"1..{MAX_MODELS} ensemble members supported")
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        hidden = int(weights[0]["w1"].shape[0])
        k1 = state_len * num_values
        if dtype not in ("bf16", "fp8", "nvfp4"):
            raise RuntimeError("dtype must be 'bf16', 'fp8' or 'nvfp4'")
        f4 = dtype == "nvfp4"
        f8 = dtype == "fp8" or f4  # NVFP4 runs the first layer on the e4m3 path
        if f4 and hidden % 256:
            raise RuntimeError("NVFP4 needs a hidden width that is a multiple of 256")
        self.dtype = dtype
        kblk = 128 if f8 else 64
        k1_pad = (onehot_columns(state_len, num_values) + kblk - 1) // kblk * kblk
        rows_pad = (int(max_rows) + 127) // 128 * 128
        self.state_len, self.state_stride, self.num_values = state_len, state_stride, num_values
        self.hidden, self.k1_pad, self.max_rows = hidden, k1_pad, int(max_rows)
        self.score_offset = float(score_offset)
        self.t: Dict[str, List[torch.Tensor]] = {k: [] for k in ("w1", "b1", "w2", "b2", "w3", "s1", "s2", "sf_w2")}
        cfg = MgbsMlpConfig()
        act_bound = 0.0
        if f8:
            for w in weights:
                w1f = np.asarray(w["w1"], dtype=np.float32).reshape(hidden, state_len, num_values)
                act_bound = max(act_bound, float((w1f.max(axis=2).sum(axis=1) + np.asarray(w["b1"], np.float32)).max()))
            act_bound = max(act_bound, 1e-6)
        act_scale = act_bound / 448.0 if f8 else 1.0
        for i, w in enumerate(weights):
            if w["w1"].shape != (hidden, k1) or w["w2"].shape != (hidden, hidden) or w["w3"].shape != (hidden,):
                raise RuntimeError("weight shapes must be w1 [H, n*V], w2 [H, H], w3 [H]")
            # first-layer weights in the kernels' one-hot column order (value-major, positions padded to eight)
            w1_f = torch.from_numpy(onehot_relayout(w["w1"], state_len, num_values, k1_pad)).to(dev)
            w2_f = torch.from_numpy(np.ascontiguousarray(w["w2"], dtype=np.float32)).to(dev)
            if f8:
                s1 = (w1_f.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
                s2w = (w2_f.abs().amax(dim=1) / 448.0).clamp_min(1e-12)
                w1 = (w1_f / s1[:, None]).to(torch.float8_e4m3fn).view(torch.uint8).contiguous()
                self.t["w1"].append(w1)
                self.t["s1"].append(s1.contiguous())
                if f4:
                    packed, sfb, w2_tscale = nvfp4_quantize_weights(np.asarray(w["w2"], dtype=np.float32))
                    self.t["w2"].append(torch.from_numpy(packed).to(dev))
                    self.t["sf_w2"].append(torch.from_numpy(sfb).to(dev))
                    act4_scale = act_bound / (6.0 * 448.0)
                    self.t["s2"].append(torch.full((hidden,), w2_tscale * act4_scale, dtype=torch.float32, device=dev))
                    cfg.sf_w2[i] = self.t["sf_w2"][i].data_ptr()
                else:
                    self.t["w2"].append((w2_f / s2w[:, None]).to(torch.float8_e4m3fn).view(torch.uint8).contiguous())
                    self.t["s2"].append((s2w * act_scale).contiguous())
                cfg.s1[i] = self.t["s1"][i].data_ptr()
                cfg.s2[i] = self.t["s2"][i].data_ptr()
            else:
                self.t["w1"].append(w1_f.to(torch.bfloat16).contiguous())
                self.t["w2"].append(w2_f.to(torch.bfloat16).contiguous())
            for k in ("b1", "b2", "w3"):
                self.t[k].append(torch.from_numpy(np.ascontiguousarray(w[k], dtype=np.float32)).to(dev))
            cfg.b3[i] = float(w["b3"])
            for k in ("w1", "b1", "w2", "b2", "w3"):
                getattr(cfg, k)[i] = self.t[k][i].data_ptr()
        # bf16: the one-hot matrix is only used by the unfused layer-1 path; fp8 has no such path
        self.x = None if f8 else torch.zeros((rows_pad, k1_pad), dtype=torch.bfloat16, device=dev)
        self.h1 = torch.zeros((rows_pad, hidden), dtype=torch.uint8 if f8 else torch.bfloat16, device=dev)
        self.q = torch.zeros((rows_pad,), dtype=torch.float32, device=dev)
        self.err = torch.zeros((1,), dtype=torch.int32, device=dev)
        self._count = torch.zeros((1,), dtype=torch.int32, device=dev)
        cfg.state_len, cfg.state_stride, cfg.num_values = state_len, state_stride, num_values
        cfg.hidden, cfg.num_models, cfg.k1_pad = hidden, len(weights), k1_pad
        cfg.max_rows = int(max_rows)
        cfg.score_offset = float(score_offset)
        cfg.x = None if f8 else self.x.data_ptr()
        cfg.h1, cfg.q, cfg.err = self.h1.data_ptr(), self.q.data_ptr(), self.err.data_ptr()
        cfg.dtype = 2 if f4 else (1 if f8 else 0)
        cfg.act_inv_scale = 1.0 / act_scale
        self.act_scale = act_scale
        self.act_bound = act_bound
        if f4:
            # packed 4-bit activations and their block factors (tiles of 128 rows x 256 columns, 4 x 512 bytes each)
            self.h1q = torch.zeros((rows_pad, hidden // 2), dtype=torch.uint8, device=dev)
            self.sf_h1 = torch.zeros((rows_pad // 128 * (hidden // 256) * 4 * 512,), dtype=torch.uint8, device=dev)
            cfg.h1q, cfg.sf_h1 = self.h1q.data_ptr(), self.sf_h1.data_ptr()
            cfg.act4_inv_global = (6.0 * 448.0) / act_bound
        self._cfg = cfg
        h = C.c_void_p()
        _lib.check(self.lib.mgbs_mlp_create(C.byref(cfg), C.byref(h)), "MLPValueScorer")
        self._h = h
        self.num_models = len(weights)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.mgbs_mlp_destroy(h)
            self._h = None

    def c_callback(self):
        """(function pointer, user pointer) for mgbs_engine_set_scorer."""
        return C.cast(self.lib.mgbs_mlp_enqueue, C.c_void_p), self._h

    def flops_per_state(self) -> int:
        """Dense multiply-add count x2 of one state through all ensemble members."""
        k1 = self.state_len * self.num_values
        return self.num_models * 2 * (k1 * self.hidden + self.hidden * self.hidden + self.hidden)

    def score(self, children: torch.Tensor) -> torch.Tensor:
        """Score rows of a [C, state_stride] uint8 CUDA tensor on the current stream; returns int32 keys [C]."""
        if children.dtype != torch.uint8 or children.dim() != 2 or children.shape[1] != self.state_stride:
            raise RuntimeError("children must be [C, state_stride] uint8")
        if children.shape[0] > self.max_rows:
            raise RuntimeError("more rows than the scorer was sized for")
        children = children.contiguous()
        self._count.fill_(children.shape[0])
        keys = torch.zeros((children.shape[0],), dtype=torch.int32, device=children.device)
        st = torch.cuda.current_stream().cuda_stream
        _lib.check(self.lib.mgbs_mlp_enqueue(self._h, children.data_ptr(), self._count.data_ptr(), keys.data_ptr(),
                                             C.c_void_p(st)), "MLPValueScorer.score")
        return keys

    def last_q(self, count: int) -> torch.Tensor:
        """Sum over ensemble members of the raw head outputs of the last call (before bias, mean and offset)."""
        return self.q[:count]

    def set_l1_mode(self, fused: bool) -> None:
        """Layer 1 with the one-hot operand built in shared memory (default) or as one-hot kernel + plain GEMM."""
        _lib.check(self.lib.mgbs_mlp_set_l1_mode(self._h, int(bool(fused))), "set_l1_mode")

    def set_head_mode(self, pair: bool) -> None:
        """Layer 2 + head on CTA pairs sharing each weight block (default) or on single CTAs (for comparison)."""
        _lib.check(self.lib.mgbs_mlp_set_head_mode(self._h, int(bool(pair))), "set_head_mode")

    def set_l1_variant(self, epilogue_warps: int = 0, pair: int = -1) -> None:
        """Layer-1 kernel variant (tuning; all variants compute the same values): 4 or 8 epilogue warps (0 = default),
        CTA pairs (-1 = default)."""
        _lib.check(self.lib.mgbs_mlp_set_l1_variant(self._h, int(epilogue_warps), int(pair)), "set_l1_variant")

    def profile(self, on: bool) -> None:
        """Record CUDA events between the scorer's kernels (eager launches only)."""
        _lib.check(self.lib.mgbs_mlp_profile(self._h, int(on)), "MLPValueScorer.profile")

    def profile_read(self) -> Dict[str, float]:
        ms = (C.c_float * 4)()
        _lib.check(self.lib.mgbs_mlp_profile_read(self._h, ms), "MLPValueScorer.profile_read")
        return {"onehot_ms": ms[0], "gemm1_ms": ms[1], "gemm2_ms": ms[2], "key_ms": ms[3]}

    def score_no_alloc(self, children: torch.Tensor, out: torch.Tensor, member: int = 0) -> int:
        """Score through the allocation-free entry point, for callers that may not allocate device memory.

        Uses ensemble member ``member`` only.  ``children`` ([C, state_stride] uint8) and ``out`` ([C] int32) are the
        caller's tensors; the library's own static device array is the only scratch.  At most NOALLOC_MAX_ROWS rows;
        larger calls raise.  Do not overlap two such calls on the GPU: they share the scratch.  Returns the GEMM
        error word (0 = clean) after waiting for the call.
        """
        if self.dtype != "bf16":
            raise RuntimeError("score_no_alloc is available for bf16 scorers only")
        if children.dtype != torch.uint8 or children.dim() != 2 or children.shape[1] != self.state_stride:
            raise RuntimeError("children must be [C, state_stride] uint8")
        if out.dtype != torch.int32 or out.numel() < children.shape[0] or not out.is_contiguous():
            raise RuntimeError("out must be a contiguous int32 tensor with one element per row")
        if not children.is_contiguous():
            raise RuntimeError("children must be contiguous")
        a = MgbsMlpNoAllocArgs()
        a.state_len, a.state_stride, a.num_values, a.hidden = self.state_len, self.state_stride, self.num_values, self.hidden
        a.score_offset = self.score_offset
        a.b3 = float(self._cfg.b3[member])
        a.w1, a.b1 = self.t["w1"][member].data_ptr(), self.t["b1"][member].data_ptr()
        a.w2, a.b2 = self.t["w2"][member].data_ptr(), self.t["b2"][member].data_ptr()
        a.w3 = self.t["w3"][member].data_ptr()
        err = C.c_int32(0)
        rc = self.lib.mgbs_mlp_score_noalloc(C.byref(a), children.data_ptr(), int(children.shape[0]), out.data_ptr(),
                                             C.byref(err), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc == -5:
            raise RuntimeError("score_no_alloc: request exceeds the library's static scratch "
                               f"(at most {NOALLOC_MAX_ROWS} rows, one-hot width 768, hidden 1024)")
        _lib.check(rc, "score_no_alloc")
        return int(err.value)

    def error_code(self) -> int:
        """0, or the code of the first bounded wait that gave up inside a GEMM kernel."""
        return int(self.err.item())


# ----------------------------------------------------------------------------------------------
# Action-value scorer (the reference's scorer contract: parents in, one value per move out)
# ----------------------------------------------------------------------------------------------


MAX_RES_BLOCKS = 4
KEY_MODES = ("q", "sigmoid_u16", "float_u16")  # MgbsQmlpConfig.key_mode


class MgbsQmlpConfig(C.Structure):
    _fields_ = [
        ("state_len", C.c_int32), ("state_stride", C.c_int32), ("num_values", C.c_int32), ("fanout", C.c_int32),
        ("hidden1", C.c_int32), ("hidden2", C.c_int32), ("num_models", C.c_int32), ("k1_pad", C.c_int32),
        ("max_parents", C.c_int64), ("score_offset", C.c_float), ("key_mode", C.c_int32),
        ("h1", C.c_void_p), ("h2", C.c_void_p), ("q", C.c_void_p), ("err", C.c_void_p),
        ("w1", C.c_void_p * MAX_MODELS), ("b1", C.c_void_p * MAX_MODELS), ("w2", C.c_void_p * MAX_MODELS),
        ("b2", C.c_void_p * MAX_MODELS), ("w3", C.c_void_p * MAX_MODELS), ("b3", C.c_void_p * MAX_MODELS),
        ("num_res_blocks", C.c_int32), ("embed_sum", C.c_int32), ("activation", C.c_int32), ("pad1", C.c_int32),
        ("h3", C.c_void_p),
        ("w1t", C.c_void_p * MAX_MODELS),
        ("wr", (C.c_void_p * MAX_MODELS) * (2 * MAX_RES_BLOCKS)), ("br", (C.c_void_p * MAX_MODELS) * (2 * MAX_RES_BLOCKS)),
    ]


_Q_SIGS = {
    "mgbs_sizeof_qmlp_config": (C.c_int, []),
    "mgbs_qmlp_create": (C.c_int, [C.POINTER(MgbsQmlpConfig), C.POINTER(C.c_void_p)]),
    "mgbs_qmlp_destroy": (C.c_int, [C.c_void_p]),
    "mgbs_qmlp_enqueue": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}
_lib.SIGNATURES.update(_Q_SIGS)


class MLPActionValueScorer:
    """Ensemble of action-value MLPs one-hot(n x V) -> hidden1 -> hidden2 -> fanout (ReLU between layers), evaluated
    once per PARENT row: candidate ``parent * fanout + move`` takes ``q[parent, move]``.  This is the reference's
    scorer contract (scorers.MLPActionScorer, scorers.py:21-36: uint8 [B, n] in, [B, fanout] out; the static
    FullBeamNice backend has the same shape, beam_engine.cpp:621-667); it costs 1/fanout of the value scorers' forward
    passes.  Weights: dicts with w1 [H1, n*V], b1, w2 [H2, H1], b2, w3 [fanout, H2], b3 [fanout]; bf16 operands, float32
    accumulation; members are averaged; keys as in the value scorers.

    Residual form (the reference's static network, scripts/static_fullbeamnice_inference.py:146-171): an optional
    ``res`` entry in each dict, a list of (wa [H2, H2], ba, wb [H2, H2], bb) per block, inserts
    x = relu(relu(x wa^T + ba) wb^T + bb + x) between hidden2 and the output layer.  ``embed_sum=True`` evaluates
    the first layer as a sum of table rows (one per position) instead of a one-hot contraction: the form for wide
    vocabularies (kernel_fullbeamnice_embed_relu, beam_kernels.cu:208-237); it is chosen automatically when the
    one-hot width exceeds what the contraction kernel holds in shared memory.  ``activation="gelu"`` (embedding-sum
    form only) and ``key_mode`` "sigmoid_u16" / "float_u16" serve the reference's MLPActionScorer /
    QuantizedActionScorer (scorers.py:21-53); see action_scorer_to_device."""

    scores_parents = True
    ONE_HOT_MAX_K = 1024  # widest one-hot first layer of the contraction kernel (16 K-blocks of 64)

    def __init__(self, weights, state_len: int, state_stride: int, num_values: int, fanout: int, max_parents: int,
                 score_offset: float = -150.0, device=None, embed_sum: Optional[bool] = None,
                 activation: str = "relu", key_mode: str = "q"):
        self.lib = _lib.load()
        for name, (res, args) in _Q_SIGS.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args
        if self.lib.mgbs_sizeof_qmlp_config() != C.sizeof(MgbsQmlpConfig):
            raise RuntimeError("structure layout mismatch between scorers.py and libmgbs_b200.so")
        if isinstance(weights, dict):
            weights = [weights]
        if not 1 <= len(weights) <= MAX_MODELS:
            raise RuntimeError(f"1..{MAX_MODELS} ensemble members supported")
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        k1 = state_len * num_values
        k1_pad = (onehot_columns(state_len, num_values) + 63) // 64 * 64
        h1, h2 = int(weights[0]["w1"].shape[0]), int(weights[0]["w2"].shape[0])
        rows_pad = (int(max_parents) + 127) // 128 * 128
        self.state_len, self.state_stride, self.num_values, self.fanout = state_len, state_stride, num_values, fanout
        self.hidden1, self.hidden2, self.num_models, self.max_parents = h1, h2, len(weights), int(max_parents)
        self._keep: List[torch.Tensor] = []
        cfg = MgbsQmlpConfig()
        cfg.state_len, cfg.state_stride, cfg.num_values, cfg.fanout = state_len, state_stride, num_values, fanout
        cfg.hidden1, cfg.hidden2, cfg.num_models, cfg.k1_pad = h1, h2, len(weights), k1_pad
        cfg.max_parents, cfg.score_offset = int(max_parents), float(score_offset)
        blocks = len(weights[0].get("res", ()))
        if blocks > MAX_RES_BLOCKS or any(len(w.get("res", ())) != blocks for w in weights):
            raise RuntimeError(f"0..{MAX_RES_BLOCKS} residual blocks, the same number in every ensemble member")
        self.num_res_blocks = blocks
        self.embed_sum = bool(k1_pad > self.ONE_HOT_MAX_K) if embed_sum is None else bool(embed_sum)
        cfg.num_res_blocks, cfg.embed_sum = blocks, int(self.embed_sum)
        if activation not in ("relu", "gelu") or key_mode not in KEY_MODES:
            raise RuntimeError("activation is relu or gelu; key_mode is one of " + ", ".join(KEY_MODES))
        if activation == "gelu" and not self.embed_sum:
            raise RuntimeError("GELU layers need embed_sum=True (the one-hot contraction kernel applies ReLU)")
        cfg.activation, cfg.key_mode = int(activation == "gelu"), KEY_MODES.index(key_mode)
        self.activation, self.key_mode = activation, key_mode

        def keep(t):
            self._keep.append(t)
            return t.data_ptr()

        def bf16(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(torch.bfloat16).contiguous()

        def f32(a):
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)

        for i, w in enumerate(weights):
            if w["w1"].shape != (h1, k1) or w["w2"].shape != (h2, h1) or w["w3"].shape != (fanout, h2):
                raise RuntimeError("weight shapes do not match the puzzle")
            for l, (wa, ba, wb, bb) in enumerate(w.get("res", ())):
                if wa.shape != (h2, h2) or wb.shape != (h2, h2) or ba.shape != (h2,) or bb.shape != (h2,):
                    raise RuntimeError("residual blocks must be square in hidden2")
                cfg.wr[2 * l][i], cfg.br[2 * l][i] = keep(bf16(wa)), keep(f32(ba))
                cfg.wr[2 * l + 1][i], cfg.br[2 * l + 1][i] = keep(bf16(wb)), keep(f32(bb))
            if self.embed_sum:
                cfg.w1t[i] = keep(bf16(np.ascontiguousarray(np.asarray(w["w1"], dtype=np.float32).T)))  # [n*V, H1]
            if self.embed_sum:
                w1 = torch.zeros((h1, 64), dtype=torch.bfloat16, device=dev)  # unused by the embedding-sum form
            else:
                w1 = bf16(onehot_relayout(w["w1"], state_len, num_values, k1_pad))
            w3 = torch.zeros((256, h2), dtype=torch.bfloat16, device=dev)
            w3[:fanout] = torch.from_numpy(np.ascontiguousarray(w["w3"], dtype=np.float32)).to(dev).to(torch.bfloat16)
            b3 = torch.zeros((256,), dtype=torch.float32, device=dev)
            b3[:fanout] = torch.from_numpy(np.ascontiguousarray(w["b3"], dtype=np.float32)).to(dev)
            cfg.w1[i], cfg.w3[i], cfg.b3[i] = keep(w1), keep(w3), keep(b3)
            cfg.w2[i] = keep(torch.from_numpy(np.ascontiguousarray(w["w2"], dtype=np.float32)).to(dev).to(torch.bfloat16).contiguous())
            cfg.b1[i] = keep(torch.from_numpy(np.ascontiguousarray(w["b1"], dtype=np.float32)).to(dev))
            cfg.b2[i] = keep(torch.from_numpy(np.ascontiguousarray(w["b2"], dtype=np.float32)).to(dev))
        self.h1 = torch.zeros((rows_pad, h1), dtype=torch.bfloat16, device=dev)
        self.h2 = torch.zeros((rows_pad, h2), dtype=torch.bfloat16, device=dev)
        if blocks:
            self.h3 = torch.zeros((rows_pad, h2), dtype=torch.bfloat16, device=dev)
            cfg.h3 = self.h3.data_ptr()
        self.q = torch.zeros((rows_pad, fanout), dtype=torch.float32, device=dev)
        self.err = torch.zeros((1,), dtype=torch.int32, device=dev)
        self._count = torch.zeros((1,), dtype=torch.int32, device=dev)
        cfg.h1, cfg.h2, cfg.q, cfg.err = self.h1.data_ptr(), self.h2.data_ptr(), self.q.data_ptr(), self.err.data_ptr()
        self._cfg = cfg
        h = C.c_void_p()
        _lib.check(self.lib.mgbs_qmlp_create(C.byref(cfg), C.byref(h)), "MLPActionValueScorer")
        self._h = h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.mgbs_qmlp_destroy(h)
            self._h = None

    def c_callback(self):
        return C.cast(self.lib.mgbs_qmlp_enqueue, C.c_void_p), self._h

    def flops_per_state(self) -> int:
        """Per CANDIDATE: one parent pass serves fanout candidates."""
        k1 = self.state_len * self.num_values
        first = self.state_len * self.hidden1 if self.embed_sum else 2 * k1 * self.hidden1  # adds only, as a sum
        per_parent = first + 2 * (self.hidden1 * self.hidden2 + 2 * self.num_res_blocks * self.hidden2 * self.hidden2
                                  + self.hidden2 * self.fanout)
        return self.num_models * per_parent // self.fanout

    def score(self, parents: torch.Tensor) -> torch.Tensor:
        """Keys [P * fanout] of all children of ``parents`` ([P, state_stride] uint8 on the device)."""
        if parents.dtype != torch.uint8 or parents.dim() != 2 or parents.shape[1] != self.state_stride:
            raise RuntimeError("parents must be [P, state_stride] uint8")
        if parents.shape[0] > self.max_parents:
            raise RuntimeError("more rows than the scorer was sized for")
        parents = parents.contiguous()
        self._count.fill_(parents.shape[0])
        keys = torch.zeros((parents.shape[0] * self.fanout,), dtype=torch.int32, device=parents.device)
        _lib.check(self.lib.mgbs_qmlp_enqueue(self._h, parents.data_ptr(), self._count.data_ptr(), keys.data_ptr(),
                                              C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                   "MLPActionValueScorer.score")
        return keys

    def last_q(self, count: int) -> torch.Tensor:
        """Action values [count, fanout] of the last call, summed over ensemble members."""
        return self.q[:count]

    def error_code(self) -> int:
        return int(self.err.item())


class MLPActionScorer(torch.nn.Module):
    """The reference's trainable action scorer with the same constructor and contract (scorers.MLPActionScorer,
    scorers.py:21-36): uint8 [B, input_dim] -> float [B, fanout]; the bytes are scaled by 1/value_scale (119 in the
    reference, its largest state value), then Linear + GELU per hidden size and a Linear to fanout.  A torch module
    for training and export; the engine runs it through action_scorer_to_device."""

    def __init__(self, input_dim: int = 120, hidden_sizes: Sequence[int] = (1024, 256), fanout: int = 24,
                 value_scale: float = 119.0):
        super().__init__()
        sizes = [int(input_dim)] + [int(h) for h in hidden_sizes]
        self.linears = torch.nn.ModuleList(torch.nn.Linear(a, b) for a, b in zip(sizes[:-1], sizes[1:]))
        self.out = torch.nn.Linear(sizes[-1], int(fanout))
        self.value_scale = float(value_scale)

    def forward(self, states_u8: torch.Tensor) -> torch.Tensor:
        x = states_u8.to(torch.float32) / self.value_scale
        for lin in self.linears:
            x = torch.nn.functional.gelu(lin(x))
        return self.out(x)


class QuantizedActionScorer(torch.nn.Module):
    """16-bit quantiser around a base scorer (scorers.QuantizedActionScorer, scorers.py:38-53): "sigmoid_u16" =
    round(sigmoid(y) * 65535), "float_u16" = round(y), clamped to 0..65535 and returned as int16 by bit pattern
    (values from 32768 come out negative).  Larger is better."""

    def __init__(self, base: torch.nn.Module, score_mode: str = "sigmoid_u16"):
        super().__init__()
        if score_mode not in ("sigmoid_u16", "float_u16"):
            raise RuntimeError("unsupported score_mode")
        self.base, self.score_mode = base, score_mode

    def forward(self, states_u8: torch.Tensor) -> torch.Tensor:
        y = self.base(states_u8)
        if self.score_mode == "sigmoid_u16":
            y = torch.sigmoid(y) * 65535.0
        q = torch.clamp(torch.round(y), 0.0, 65535.0).to(torch.int32)
        return torch.where(q >= 32768, q - 65536, q).to(torch.int16)


def make_default_mlp_scorer(hidden_sizes: Sequence[int] = (1024, 256), fanout: int = 24, input_dim: int = 120,
                            value_scale: float = 119.0) -> torch.nn.Module:
    """make_default_mlp_scorer (scorers.py:56-57): sigmoid-quantised MLPActionScorer."""
    return QuantizedActionScorer(MLPActionScorer(input_dim, hidden_sizes, fanout, value_scale))


def action_scorer_to_device(module: torch.nn.Module, state_len: int, state_stride: int, num_values: int,
                            max_parents: int, device=None) -> "MLPActionValueScorer":
    """Device scorer for an MLPActionScorer or a QuantizedActionScorer around one (two hidden layers, each a
    multiple of 256 wide).  The dense first layer on bytes scaled by 1/value_scale is a sum of table rows
    ``W1[:, pos] * value / value_scale`` - one per position - so it runs on the embedding-sum kernel; hidden layers
    use GELU; a quantised wrapper selects the matching key mode (key = 65535 - its 16-bit score), a bare
    MLPActionScorer gives keys uint32(clamp(y, 0, 300) * 256 + 0.5)."""
    key_mode = "q"
    base = module
    if isinstance(module, QuantizedActionScorer):
        key_mode, base = module.score_mode, module.base
    if not isinstance(base, MLPActionScorer) or len(base.linears) != 2:
        raise RuntimeError("action_scorer_to_device takes an MLPActionScorer with two hidden layers")
    if base.linears[0].in_features != state_len:
        raise RuntimeError(f"the scorer reads {base.linears[0].in_features} bytes per state, the puzzle has {state_len}")
    w1 = _np(base.linears[0].weight)  # [H1, n]
    values = (np.arange(num_values, dtype=np.float32) / np.float32(base.value_scale))
    table = (w1.T[:, None, :] * values[None, :, None]).reshape(state_len * num_values, w1.shape[0])  # row = pos*V + v
    w = {"w1": np.ascontiguousarray(table.T), "b1": _np(base.linears[0].bias),
         "w2": _np(base.linears[1].weight), "b2": _np(base.linears[1].bias),
         "w3": _np(base.out.weight), "b3": _np(base.out.bias)}
    return MLPActionValueScorer(w, state_len, state_stride, num_values, base.out.out_features, max_parents,
                                score_offset=0.0, device=device, embed_sum=True, activation="gelu", key_mode=key_mode)


def _np(t) -> np.ndarray:
    return t.detach().float().cpu().numpy() if isinstance(t, torch.Tensor) else np.asarray(t, dtype=np.float32)


def fold_bn_linear(weight, bias, bn_weight, bn_bias, running_mean, running_var, eps: float = 1e-5):
    """Inference-form batch norm folded into the linear layer before it (float32): W' = W * s per output row,
    b' = (b - mean) * s + beta with s = gamma / sqrt(var + eps) (_fold_bn_linear,
    scripts/static_fullbeamnice_inference.py:59-71)."""
    scale = (_np(bn_weight) / np.sqrt(_np(running_var) + np.float32(eps))).astype(np.float32)
    w = (_np(weight) * scale[:, None]).astype(np.float32)
    b = ((_np(bias) - _np(running_mean)) * scale + _np(bn_bias)).astype(np.float32)
    return w, b


def static_weights_from_state_dict(sd: Dict[str, Any], num_res_blocks: int, state_len: int, num_classes: int,
                                   state_size: Optional[int] = None, class_pad: Optional[int] = None,
                                   action_perm: Optional[Sequence[int]] = None) -> Dict[str, Any]:
    """The reference's static weight dictionary from a trained module's state dict (load_static_weights,
    scripts/static_fullbeamnice_inference.py:74-143): batch norms folded into input_layer, hidden_layer and every
    residual_blocks.{i}.fc{1,2}; matrices transposed to [in, out]; the embedding re-laid from ``num_classes`` rows
    per position to ``class_pad`` rows per position over ``state_size`` positions (the reference pads 120 x 120 to
    128 x 128), new rows zero."""
    state_size = int(state_size or state_len)
    class_pad = int(class_pad or num_classes)
    embed = _np(sd["input_layer.weight"])
    hd1 = _np(sd["input_layer.bias"]).shape[0]
    if embed.shape[0] == hd1 and embed.shape[1] == state_len * num_classes:
        embed = np.ascontiguousarray(embed.T)  # stored [out, in]
    if embed.shape != (state_len * num_classes, hd1):
        raise RuntimeError(f"input_layer.weight has shape {embed.shape}, expected {(state_len * num_classes, hd1)}")
    table = np.zeros((state_size * class_pad, hd1), dtype=np.float32)
    for pos in range(state_len):
        table[pos * class_pad: pos * class_pad + num_classes] = embed[pos * num_classes: (pos + 1) * num_classes]
    s1 = (_np(sd["bn1.weight"]) / np.sqrt(_np(sd["bn1.running_var"]) + np.float32(1e-5))).astype(np.float32)
    out: Dict[str, Any] = {
        "embed_w_t": table * s1[None, :],
        "embed_bias": (_np(sd["input_layer.bias"]) - _np(sd["bn1.running_mean"])) * s1 + _np(sd["bn1.bias"]),
    }
    hw, hb = fold_bn_linear(sd["hidden_layer.weight"], sd["hidden_layer.bias"], sd["bn2.weight"], sd["bn2.bias"],
                            sd["bn2.running_mean"], sd["bn2.running_var"])
    out["hidden_w_t"], out["hidden_bias"] = np.ascontiguousarray(hw.T), hb
    for b in range(int(num_res_blocks)):
        pre = f"residual_blocks.{b}"
        for fc, bn in (("fc1", "bn1"), ("fc2", "bn2")):
            w, bias = fold_bn_linear(sd[f"{pre}.{fc}.weight"], sd[f"{pre}.{fc}.bias"], sd[f"{pre}.{bn}.weight"],
                                     sd[f"{pre}.{bn}.bias"], sd[f"{pre}.{bn}.running_mean"], sd[f"{pre}.{bn}.running_var"])
            out[f"res{b}_{fc}_w_t"], out[f"res{b}_{fc}_bias"] = np.ascontiguousarray(w.T), bias
    out["out_w_t"] = np.ascontiguousarray(_np(sd["output_layer.weight"]).T)
    out["out_bias"] = _np(sd["output_layer.bias"])
    outputs = out["out_bias"].shape[0]
    out["action_perm"] = np.asarray(action_perm if action_perm is not None else np.arange(outputs), dtype=np.int64)
    out["state_size"], out["num_classes"] = state_size, class_pad
    out["score_scale"], out["score_bias"] = 1024.0, 65535.0
    return out


def fullbeamnice_scorer_from_static_weights(weights: Dict[str, Any], state_len: int, state_stride: int, fanout: int,
                                            max_parents: int, score_offset: float = 0.0, device=None,
                                            embed_sum: Optional[bool] = None) -> "MLPActionValueScorer":
    """Action-value scorer from the reference's static weight dictionary (keys embed_w_t, embed_bias, hidden_w_t,
    hidden_bias, res{i}_fc{1,2}_w_t / _bias, out_w_t, out_bias, action_perm, state_size, num_classes;
    StaticFullBeamNiceWeights, scripts/static_fullbeamnice_inference.py:36-56, consumed by
    FullBeamNiceStaticBackend, beam_engine.cpp:556-619).

    The dictionary's tables are [in, out]; they are transposed here.  Positions past ``state_len`` (the reference
    stores 120-byte states in 128 positions, the extra ones holding value 0) contribute the constant row
    ``embed_w_t[pos * num_classes]``, which is folded into the first bias.  The output columns are reordered by
    ``action_perm`` (q_current = q[:, action_perm], static_forward_scores :174-178), so column m is move m of the
    engine.  Keys are uint32(clamp(q - score_offset, 0, 300) * 256 + 0.5) as in
    kernel_fullbeamnice_q_to_score_key_ring (beam_kernels.cu:326-346); the reference uses offset 0."""
    size, classes = int(weights["state_size"]), int(weights["num_classes"])
    if state_len > size:
        raise RuntimeError(f"the weights cover {size} positions, the puzzle has {state_len}")
    table = _np(weights["embed_w_t"])
    h1 = table.shape[1]
    if table.shape[0] != size * classes:
        raise RuntimeError(f"embed_w_t has {table.shape[0]} rows, expected state_size * num_classes = {size * classes}")
    b1 = _np(weights["embed_bias"]).astype(np.float32).copy()
    for pos in range(state_len, size):
        b1 += table[pos * classes]
    perm = np.asarray(_np(weights["action_perm"]), dtype=np.int64)
    if perm.shape[0] != fanout or sorted(perm.tolist()) != list(range(fanout)):
        raise RuntimeError("action_perm must be a permutation of the engine's moves")
    res = []
    b = 0
    while f"res{b}_fc1_w_t" in weights:
        res.append((np.ascontiguousarray(_np(weights[f"res{b}_fc1_w_t"]).T), _np(weights[f"res{b}_fc1_bias"]),
                    np.ascontiguousarray(_np(weights[f"res{b}_fc2_w_t"]).T), _np(weights[f"res{b}_fc2_bias"])))
        b += 1
    w = {
        "w1": np.ascontiguousarray(table[: state_len * classes].T), "b1": b1,
        "w2": np.ascontiguousarray(_np(weights["hidden_w_t"]).T), "b2": _np(weights["hidden_bias"]),
        "w3": np.ascontiguousarray(_np(weights["out_w_t"]).T[perm]), "b3": _np(weights["out_bias"])[perm],
        "res": res,
    }
    return MLPActionValueScorer(w, state_len, state_stride, classes, fanout, max_parents, score_offset=score_offset,
                                device=device, embed_sum=embed_sum)


# ----------------------------------------------------------------------------------------------
# Transformer value scorer
# ----------------------------------------------------------------------------------------------

TF_MAX_ENCODERS = 4
TF_MAX_LAYERS = 8
_LAYER_FIELDS = ("ln1_g", "ln1_b", "wqkv", "bqkv", "wo", "bo", "ln2_g", "ln2_b", "w1", "b1", "w2", "b2")
_LAYER_BF16 = {"wqkv", "wo", "w1", "w2"}
E4M3_MAX = 448.0


class MgbsTfLayer(C.Structure):
    _fields_ = ([(name, C.c_void_p) for name in _LAYER_FIELDS]
                + [(name, C.c_void_p) for name in ("cs_qkv", "cs_o", "cs_1", "cs_2")]
                + [(name, C.c_float) for name in ("inv_y1", "inv_att", "inv_y2", "inv_hid")])


class MgbsTfConfig(C.Structure):
    _fields_ = [
        ("state_len", C.c_int32), ("state_stride", C.c_int32), ("num_values", C.c_int32), ("d_model", C.c_int32),
        ("heads", C.c_int32), ("ffn", C.c_int32), ("layers", C.c_int32), ("encoders", C.c_int32),
        ("max_states", C.c_int64), ("micro_batch", C.c_int64), ("score_offset", C.c_float),
        ("b_head", C.c_float * TF_MAX_ENCODERS),
        ("tok_emb", C.c_void_p * TF_MAX_ENCODERS), ("pos_emb", C.c_void_p * TF_MAX_ENCODERS),
        ("lnf_g", C.c_void_p * TF_MAX_ENCODERS), ("lnf_b", C.c_void_p * TF_MAX_ENCODERS),
        ("w_head", C.c_void_p * TF_MAX_ENCODERS),
        ("layer", (MgbsTfLayer * TF_MAX_LAYERS) * TF_MAX_ENCODERS),
        ("x", C.c_void_p), ("y", C.c_void_p), ("qkv", C.c_void_p), ("att", C.c_void_p), ("hid", C.c_void_p),
        ("q", C.c_void_p), ("err", C.c_void_p), ("dtype", C.c_int32), ("reserved", C.c_int32),
    ]


_TF_SIGS = {
    "mgbs_sizeof_tf_config": (C.c_int, []),
    "mgbs_tf_create": (C.c_int, [C.POINTER(MgbsTfConfig), C.POINTER(C.c_void_p)]),
    "mgbs_tf_destroy": (C.c_int, [C.c_void_p]),
    "mgbs_tf_enqueue": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}
_lib.SIGNATURES.update(_TF_SIGS)


class TransformerValueScorer:
    """Ensemble of pre-LayerNorm transformer encoders scoring child states (see puzzles.transformer_weights for the
    weight layout): d_model 256, 8 heads, GELU feed-forward, mean pooling, scalar head.  bf16 GEMM operands with fp32
    accumulation on the tcgen05 tensor cores, fp32 residual stream; states go through in micro-batches of
    ``micro_batch`` (the reference's B_MICRO knob).

    ``dtype="fp8"`` stores the four matrices of every layer as e4m3 with one scale per output row and feeds the GEMMs
    e4m3 activations (LayerNorm output, attention output, GELU output) with one scale per tensor.  The activation
    scales come from bounds that hold for every input (a LayerNorm row has L2 norm 16 before its gain, so
    |row . w| <= (16 max|gain| + |shift|) |w|), not from calibration data; q, k, v stay bf16 for the attention
    kernel.  ``dtype="nvfp4_weights"`` rounds the same matrices to the NVFP4 grid and runs them on the bf16 path."""

    def __init__(self, encoders: Sequence[Dict], state_len: int, state_stride: int, num_values: int, max_rows: int,
                 micro_batch: int = 32768, score_offset: float = -150.0, device=None, dtype: str = "bf16"):
        self.lib = _lib.load()
        for name, (res, args) in _TF_SIGS.items():
            fn = getattr(self.lib, name)
            fn.restype, fn.argtypes = res, args
        if self.lib.mgbs_sizeof_tf_config() != C.sizeof(MgbsTfConfig):
            raise RuntimeError("structure layout mismatch between scorers.py and libmgbs_b200.so")
        if isinstance(encoders, dict):
            encoders = [encoders]
        if not 1 <= len(encoders) <= TF_MAX_ENCODERS:
            raise RuntimeError(f"1..{TF_MAX_ENCODERS} encoders supported")
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        d = int(encoders[0]["tok_emb"].shape[1])
        layers = len(encoders[0]["layers"])
        ffn = int(encoders[0]["layers"][0]["w1"].shape[0])
        micro_batch = int(min(micro_batch, max_rows))
        rows_pad = (micro_batch * state_len + 127) // 128 * 128
        self.state_len, self.state_stride, self.num_values = state_len, state_stride, num_values
        self.max_rows, self.micro_batch, self.score_offset = int(max_rows), micro_batch, float(score_offset)
        self.d_model, self.layers, self.ffn, self.num_models = d, layers, ffn, len(encoders)
        self._keep: List[torch.Tensor] = []

        def f32(a):
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)
            self._keep.append(t)
            return t.data_ptr()

        def bf16(a):
            t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(torch.bfloat16).contiguous()
            self._keep.append(t)
            return t.data_ptr()

        if dtype not in ("bf16", "fp8", "nvfp4_weights"):
            raise RuntimeError("dtype must be 'bf16', 'fp8' or 'nvfp4_weights'")
        self.dtype = dtype
        fp8 = dtype == "fp8"
        if dtype == "nvfp4_weights":
            # the four matrices of every layer rounded to the NVFP4 grid (E2M1 elements, E4M3 block-16 factors, one
            # tensor scale) and fed to the bf16 GEMMs: these kernels are bound by activation bytes (K = 256), so the
            # weights' storage format does not change their time; what this gives is the numerics of NVFP4 weights
            encoders = [dict(w, layers=[dict(L, **{k: nvfp4_round_weights(L[k]) for k in _LAYER_BF16}) for L in w["layers"]])
                        for w in encoders]

        def e4m3(w, act_scale):
            """Rows of w as e4m3 with per-row scales; returns (weights ptr, column-scale ptr)."""
            w = torch.from_numpy(np.ascontiguousarray(w, dtype=np.float32))
            ws = (w.abs().amax(dim=1).clamp_min(1e-30) / E4M3_MAX).to(torch.float32)
            q8 = (w / ws[:, None]).to(torch.float8_e4m3fn).contiguous().to(dev)
            cs = (ws * float(act_scale)).to(dev)
            self._keep += [q8, cs]
            return q8.data_ptr(), cs.data_ptr()

        def ln_bound(gain, shift):
            """Upper bound of the L2 norm of a LayerNorm output row of width d."""
            return float(np.sqrt(d) * np.abs(gain).max() + np.linalg.norm(shift))

        def out_bound(w, b, in_norm):
            """Upper bound of |x . w_row + b| over rows, for |x|_2 <= in_norm."""
            return float((np.linalg.norm(np.asarray(w, dtype=np.float64), axis=1) * in_norm + np.abs(b)).max())

        cfg = MgbsTfConfig()
        cfg.dtype = 1 if fp8 else 0
        cfg.state_len, cfg.state_stride, cfg.num_values = state_len, state_stride, num_values
        cfg.d_model, cfg.heads, cfg.ffn, cfg.layers, cfg.encoders = d, 8, ffn, layers, len(encoders)
        cfg.max_states, cfg.micro_batch, cfg.score_offset = int(max_rows), micro_batch, float(score_offset)
        for e, w in enumerate(encoders):
            if w["tok_emb"].shape != (num_values, d) or w["pos_emb"].shape[0] < state_len or len(w["layers"]) != layers:
                raise RuntimeError("encoder weight shapes do not match the puzzle")
            cfg.b_head[e] = float(w["b_head"])
            cfg.tok_emb[e], cfg.pos_emb[e] = f32(w["tok_emb"]), f32(w["pos_emb"][:state_len])
            cfg.lnf_g[e], cfg.lnf_b[e], cfg.w_head[e] = f32(w["lnf_g"]), f32(w["lnf_b"]), f32(w["w_head"])
            for li, L in enumerate(w["layers"]):
                dst = cfg.layer[e][li]
                for name in _LAYER_FIELDS:
                    if not (fp8 and name in _LAYER_BF16):
                        setattr(dst, name, bf16(L[name]) if name in _LAYER_BF16 else f32(L[name]))
                if fp8:
                    n1, n2 = ln_bound(L["ln1_g"], L["ln1_b"]), ln_bound(L["ln2_g"], L["ln2_b"])
                    # element bounds: LN rows by their norm, attention output by the largest |v|, GELU by |input|
                    s_y1, s_y2 = n1 / E4M3_MAX, n2 / E4M3_MAX
                    s_att = out_bound(L["wqkv"][2 * d:], L["bqkv"][2 * d:], n1) / E4M3_MAX
                    s_hid = out_bound(L["w1"], L["b1"], n2) / E4M3_MAX
                    dst.wqkv, dst.cs_qkv = e4m3(L["wqkv"], s_y1)
                    dst.wo, dst.cs_o = e4m3(L["wo"], s_att)
                    dst.w1, dst.cs_1 = e4m3(L["w1"], s_y2)
                    dst.w2, dst.cs_2 = e4m3(L["w2"], s_hid)
                    dst.inv_y1, dst.inv_att, dst.inv_y2, dst.inv_hid = 1 / s_y1, 1 / s_att, 1 / s_y2, 1 / s_hid
        act = torch.uint8 if fp8 else torch.bfloat16
        self.x = torch.zeros((rows_pad, d), dtype=torch.float32, device=dev)
        self.y = torch.zeros((rows_pad, d), dtype=act, device=dev)
        self.qkv = torch.zeros((rows_pad, 3 * d), dtype=torch.bfloat16, device=dev)
        self.att = torch.zeros((rows_pad, d), dtype=act, device=dev)
        self.hid = torch.zeros((rows_pad, ffn), dtype=act, device=dev)
        self.q = torch.zeros((int(max_rows),), dtype=torch.float32, device=dev)
        self.err = torch.zeros((1,), dtype=torch.int32, device=dev)
        self._count = torch.zeros((1,), dtype=torch.int32, device=dev)
        cfg.x, cfg.y, cfg.qkv, cfg.att, cfg.hid = (t.data_ptr() for t in (self.x, self.y, self.qkv, self.att, self.hid))
        cfg.q, cfg.err = self.q.data_ptr(), self.err.data_ptr()
        self._cfg = cfg
        h = C.c_void_p()
        _lib.check(self.lib.mgbs_tf_create(C.byref(cfg), C.byref(h)), "TransformerValueScorer")
        self._h = h

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            self.lib.mgbs_tf_destroy(h)
            self._h = None

    def c_callback(self):
        return C.cast(self.lib.mgbs_tf_enqueue, C.c_void_p), self._h

    def flops_per_state(self) -> int:
        d, t, f = self.d_model, self.state_len, self.ffn
        per_layer = 2 * t * (3 * d * d + d * d + 2 * d * f) + 2 * 2 * t * t * d
        return self.num_models * self.layers * per_layer

    def score(self, children: torch.Tensor) -> torch.Tensor:
        if children.dtype != torch.uint8 or children.dim() != 2 or children.shape[1] != self.state_stride:
            raise RuntimeError("children must be [C, state_stride] uint8")
        if children.shape[0] > self.max_rows:
            raise RuntimeError("more rows than the scorer was sized for")
        children = children.contiguous()
        self._count.fill_(children.shape[0])
        keys = torch.zeros((children.shape[0],), dtype=torch.int32, device=children.device)
        _lib.check(self.lib.mgbs_tf_enqueue(self._h, children.data_ptr(), self._count.data_ptr(), keys.data_ptr(),
                                            C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                   "TransformerValueScorer.score")
        return keys

    def last_q(self, count: int) -> torch.Tensor:
        return self.q[:count]

    def error_code(self) -> int:
        return int(self.err.item())
