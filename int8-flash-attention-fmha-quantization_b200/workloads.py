"""Seeded synthetic inputs for the five benchmark shapes of the INT8 attention forward path.

No public dataset backs this path: the reference project draws its test data from a seeded
generator (test_fmha_i8.cpp:43-111), so every workload here is synthetic as well.  Shapes and value
distributions:

  C1  B=1   H=2  S=64     D=64   Q,K,V ~ N(0,1)                no padding
  C2  B=32  H=12 S=512    D=64   Q,K,V ~ N(0,1)                valid length per batch in {256,...,512} step 64
  C3  B=8   H=32 S=2048   D=128  Q,K ~ N(0,1), V ~ N(0,0.5)    no padding       (0.5 = standard deviation)
  C4  B=1   H=32 S=16384  D=128  N(0,1), 1 % of Q and K x8     valid length 15360
  C5  B=256 H=16 S=256    D=64   Q,K,V ~ N(0,1)                valid length per batch in {64,...,256} step 64

The wire format of the padding mask keeps the reference's polarity: byte != 0 means the key is
masked out (inc/cpuSoftmax.hpp:9,24; inc/fmha_i8.cuh:189-192).  A valid length L is therefore
encoded as mask[b, s] = (s >= L).

Per-tensor symmetric quantisation follows inc/utils.hpp:23-39: amax = max|x|,
q = clamp(floor(x * 127/amax + 0.5), -127, 127).
"""
from dataclasses import dataclass, field
from typing import Optional, Tuple

import numpy as np


@dataclass(frozen=True)
class Workload:
    name: str
    B: int
    H: int
    S: int
    D: int
    v_std: float = 1.0
    outlier_frac: float = 0.0
    outlier_gain: float = 8.0
    valid_choices: Optional[Tuple[int, ...]] = None  # None => no padding

    @property
    def ops(self) -> float:
        """Algorithmic work of one forward pass: 4*B*H*S^2*D (two dense contractions, no mask discount)."""
        return 4.0 * self.B * self.H * self.S * self.S * self.D

    @property
    def bytes(self) -> float:
        """Algorithmic HBM traffic: Q,K,V read + O written + mask read."""
        return 4.0 * self.B * self.H * self.S * self.D + self.B * self.S

    def with_batch(self, B):
        return Workload(self.name, B, self.H, self.S, self.D, self.v_std, self.outlier_frac, self.outlier_gain,
                        self.valid_choices)


CONFIGS = {
    "C1": Workload("C1", 1, 2, 64, 64),
    "C2": Workload("C2", 32, 12, 512, 64, valid_choices=(256, 320, 384, 448, 512)),
    "C3": Workload("C3", 8, 32, 2048, 128, v_std=0.5),
    "C4": Workload("C4", 1, 32, 16384, 128, outlier_frac=0.01, valid_choices=(15360,)),
    "C5": Workload("C5", 256, 16, 256, 64, valid_choices=(64, 128, 192, 256)),
}


def valid_lengths(w: Workload, seed: int) -> np.ndarray:
    if w.valid_choices is None:
        return np.full(w.B, w.S, np.int64)
    rng = np.random.Generator(np.random.Philox(key=seed + 7))
    return rng.choice(np.asarray(w.valid_choices, np.int64), size=w.B)


def mask_from_valid(valid: np.ndarray, S: int) -> np.ndarray:
    """int8 [B,S]; 1 where the key is padding (s >= valid length)."""
    return (np.arange(S)[None, :] >= np.asarray(valid)[:, None]).astype(np.int8)


def quantize_np(x: np.ndarray):
    """Per-tensor symmetric int8, arithmetic of inc/utils.hpp:23-39 (float32 scale, double +0.5)."""
    x = np.asarray(x, np.float32)
    amax = np.float32(np.max(np.abs(x)))
    scale = np.float32(127.0) / amax
    f = (x * scale).astype(np.float32)
    q = np.floor((f.astype(np.float64) + 0.5).astype(np.float32))
    return np.clip(q, -127, 127).astype(np.int8), float(amax)


def make_fp32_np(w: Workload, seed: int = 2023):
    """fp32 Q,K,V [B,H,S,D] and the int8 mask [B,S], from counter-based streams (one per tensor)."""
    shape = (w.B, w.H, w.S, w.D)
    out = []
    for i, std in enumerate((1.0, 1.0, w.v_std)):
        rng = np.random.Generator(np.random.Philox(key=seed * 16 + i))
        x = rng.standard_normal(shape, dtype=np.float32)
        if std != 1.0:
            x *= np.float32(std)
        if w.outlier_frac > 0 and i < 2:
            sel = np.random.Generator(np.random.Philox(key=seed * 16 + 8 + i)).random(shape, dtype=np.float32)
            x = np.where(sel < w.outlier_frac, x * np.float32(w.outlier_gain), x).astype(np.float32)
        out.append(x)
    mask = mask_from_valid(valid_lengths(w, seed), w.S)
    return out[0], out[1], out[2], mask


# ---------------------------------------------------------------------------------------------
# Device-side generation for the large shapes (benchmark / full-size property tests).  torch is
# plumbing here: it owns the device memory and the random stream, nothing on the timed path.
# ---------------------------------------------------------------------------------------------
def quantize_torch(x):
    import torch
    amax = x.abs().max()
    scale = (torch.tensor(127.0, dtype=torch.float32, device=x.device) / amax)
    f = x * scale
    q = torch.floor((f.double() + 0.5).float())
    return q.clamp_(-127, 127).to(torch.int8), float(amax)


def make_int8_torch(w: Workload, seed: int, device, want_fp32: bool = False):
    """Returns dict(q8,k8,v8 int8 [B,H,S,D], mask int8 [B,S], amax=(q,k,v), valid=...) on `device`.
    Tensors are generated and quantised one at a time so that C3/C4 need < 1 GB of fp32 scratch."""
    import torch
    g = torch.Generator(device=device)
    shape = (w.B, w.H, w.S, w.D)
    res, amax, fp = {}, [], {}
    for i, (name, std) in enumerate((("q", 1.0), ("k", 1.0), ("v", w.v_std))):
        g.manual_seed(seed * 16 + i)
        x = torch.randn(shape, generator=g, device=device, dtype=torch.float32)
        if std != 1.0:
            x.mul_(std)
        if w.outlier_frac > 0 and i < 2:
            g.manual_seed(seed * 16 + 8 + i)
            sel = torch.rand(shape, generator=g, device=device, dtype=torch.float32) < w.outlier_frac
            x = torch.where(sel, x * w.outlier_gain, x)
        q8, a = quantize_torch(x)
        res[name + "8"] = q8
        amax.append(a)
        if want_fp32:
            fp[name] = x
        else:
            del x
    valid = valid_lengths(w, seed)
    res["mask"] = torch.from_numpy(mask_from_valid(valid, w.S)).to(device)
    res["amax"] = tuple(amax)
    res["valid"] = valid
    res.update(fp)
    return res


def fp32_attention_torch(q, k, v, mask, chunk_heads: int = 4):
    """fp32 attention on the device, used only to calibrate o_amax for shapes whose CPU golden
    would need tens of GB (C3, C4).  mask: int8 [B,S], non-zero = masked key."""
    import torch
    B, H, S, D = q.shape
    o_absmax = 0.0
    out = torch.empty_like(q)
    keep = (mask == 0)[:, None, None, :]  # [B,1,1,S], True = attend
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        for h0 in range(0, H, chunk_heads):
            h1 = min(H, h0 + chunk_heads)
            o = torch.nn.functional.scaled_dot_product_attention(q[:, h0:h1], k[:, h0:h1], v[:, h0:h1], attn_mask=keep)
            out[:, h0:h1] = o
            o_absmax = max(o_absmax, float(o.abs().max()))
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return out, o_absmax
