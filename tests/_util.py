"""Shared helpers of the test-suite: seeded inputs with the value distributions of the benchmark
configurations, and conversion of the library's storage layouts to logical (row, block) order."""
import importlib.util
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


def make_qkv(B, Hq, Hkv, Nq, Nk, D, seed=0, k_offset_std=2.0, v_outlier_frac=0.0, layout="HND", device="cpu"):
    """Q, K, V ~ N(0,1) in bf16; K gets a per-(head, channel) offset ~ N(0, k_offset_std^2) shared by
    all tokens (the channel outliers K smoothing removes); a fraction of V channels is scaled by 8.
    Generated on the CPU generator so that every device sees the same values."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, Nq, D, generator=g)
    k = torch.randn(B, Hkv, Nk, D, generator=g)
    v = torch.randn(B, Hkv, Nk, D, generator=g)
    if k_offset_std > 0:
        k = k + k_offset_std * torch.randn(B, Hkv, 1, D, generator=g)
    if v_outlier_frac > 0:
        n = max(1, int(round(D * v_outlier_frac)))
        for b in range(B):
            for h in range(Hkv):
                idx = torch.randperm(D, generator=g)[:n]
                v[b, h, :, idx] *= 8
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    if layout == "NHD":
        q, k, v = (t.transpose(1, 2).contiguous() for t in (q, k, v))
    return q.to(device), k.to(device), v.to(device)


def sf_atoms_to_logical(sf_atoms: np.ndarray, rows: int) -> np.ndarray:
    """[..., A, 512] scale atoms (A atoms of 4 blocks each) -> [..., rows, 4*A] logical scale bytes."""
    A = sf_atoms.shape[-2]
    r = np.arange(rows)[:, None]
    b = np.arange(4 * A)[None, :]
    off = (b // 4) * 512 + (r % 32) * 16 + (r // 32) * 4 + (b % 4)
    flat = sf_atoms.reshape(*sf_atoms.shape[:-2], A * 512)
    return flat[..., off]


def unpack_rows(codes: torch.Tensor, sf: torch.Tensor):
    """Q/K buffers [B,H,T,128,D/2], [B,H,T,D/64,512] -> codes [B,H,T*128,D/2], sf [B,H,T*128,D/16]."""
    c = codes.cpu().numpy()
    B, H, T = c.shape[:3]
    s = sf_atoms_to_logical(sf.cpu().numpy(), 128)            # [B,H,T,128,D/16]
    return c.reshape(B, H, T * 128, -1), s.reshape(B, H, T * 128, -1)


def unpack_vt(codes: torch.Tensor, sf: torch.Tensor):
    """V^T buffers [B,H,T,D,64], [B,H,T,2,512] -> codes [B,H,D,T*64], sf [B,H,D,T*8]."""
    c = codes.cpu().numpy()
    B, H, T, D, _ = c.shape
    s = sf_atoms_to_logical(sf.cpu().numpy(), D)              # [B,H,T,D,8]
    c = np.transpose(c, (0, 1, 3, 2, 4)).reshape(B, H, D, T * 64)
    s = np.transpose(s, (0, 1, 3, 2, 4)).reshape(B, H, D, T * 8)
    return c, s


def load_reference_quant():
    """The reference's own CUDA quantisation kernels, compiled for sm_100a by oracle/build_ref.py."""
    so = ROOT / "oracle" / "_ref" / "sage_ref_quant_cuda.so"
    if not so.exists():
        return None
    spec = importlib.util.spec_from_file_location("sage_ref_quant_cuda", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bf16_np(x: torch.Tensor) -> np.ndarray:
    return x.detach().float().cpu().numpy()
