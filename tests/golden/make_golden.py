"""Generate golden vectors from the reference's own Python code (run in a container that has the
reference checkout; the output ``.npz`` files are committed, the checkout is not needed later).

    python tests/golden/make_golden.py [/path/to/reference]

``sageattn4/api.py`` cannot be imported as a module (it imports two compiled CUDA extensions at the
top), so the pure-PyTorch functions are lifted out of its syntax tree and executed unchanged:
``round_to_blockscaled_fp4`` / ``round_to_token_blockscaled_fp4`` (api.py:77-110).
Outputs:

* ``quant_emulation.npz``  - seeded inputs (bf16 bit patterns) incl. every E2M1 tie point, and the
  reference emulation's de-quantised result for row-wise and token-wise (transposed V) blocks.
* ``pack_emulation.npz`` - the fork's K-packing preprocessing (``preprocess_qkv``, api.py:112-205, run
  unchanged on CPU with per_block_mean=True; its Triton group-mean helper, which needs a GPU, is
  replaced by the same arithmetic in PyTorch): packed K, lambda, packed V and delta_s for a seeded
  ragged input and for the s128 real-activation fixture.
* ``llama_fixture_qkv.npz`` - the reference's real-activation test inputs
  (``tests/fixtures/llama3p1_8b_instruct_l16_h30_s256_qkv.pt`` and ``..._h15_s128_qkv.pt``; inputs
  only, the reference commits no expected outputs) as bf16 bit patterns, plus the reference
  emulation applied to the smoothed K and to V, and the fp32 SDPA result that the reference's
  only test compares against (tests/test.py:27-47).
"""
import ast
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def lift(api_path: Path, names, extra=None):
    tree = ast.parse(api_path.read_text())
    body = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    mod = ast.Module(body=body, type_ignores=[])
    ns = {"torch": torch}
    ns.update(extra or {})
    exec(compile(mod, str(api_path), "exec"), ns)
    return [ns[n] for n in names]


def bits(x: torch.Tensor) -> np.ndarray:
    return x.contiguous().view(torch.int16).numpy().view(np.uint16)


def main(ref_root: str):
    ref = Path(ref_root) / "sageattention3_blackwell"
    rtb, rttb = lift(ref / "sageattn4" / "api.py",
                     ["round_to_blockscaled_fp4", "round_to_token_blockscaled_fp4"])

    g = torch.Generator().manual_seed(0)
    rows = [torch.zeros(16)]
    # (1) every E2M1 midpoint, at several block scales, both signs
    ties = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.0, 6.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 5.5])
    for s in [1.0, 0.5, 2.0, 0.375, 1.75, 448.0 / 64, 2.0 ** -6, 2.0 ** -9]:
        rows.append(ties * s)
        rows.append(-(ties * s))
    # (2) random normal, heavy-tailed and tiny/huge magnitude rows
    rows += list(torch.randn(64, 16, generator=g))
    rows += list(torch.randn(32, 16, generator=g) * torch.randn(32, 1, generator=g).exp() * 4)
    rows += list(torch.randn(16, 16, generator=g) * 1e-3)
    rows += list(torch.randn(16, 16, generator=g) * 300)
    x = torch.stack(rows).to(torch.bfloat16)
    x = x.reshape(-1, 128) if x.numel() % 128 == 0 else x[: (x.shape[0] // 8) * 8].reshape(-1, 128)
    y = rtb(x)
    # token-wise: [tokens=32, channels=24] blocks along tokens
    xt = (torch.randn(2, 3, 32, 24, generator=g) * 3).to(torch.bfloat16)
    yt = rttb(xt)
    np.savez_compressed(HERE / "quant_emulation.npz", x=bits(x), y=bits(y), xt=bits(xt), yt=bits(yt))
    print("quant_emulation.npz", x.shape, xt.shape)

    out = {}
    for tag, name in [("s256", "llama3p1_8b_instruct_l16_h30_s256_qkv.pt"),
                      ("s128", "llama3p1_8b_instruct_l16_h15_s128_qkv.pt")]:
        d = torch.load(ref / "tests" / "fixtures" / name, map_location="cpu")
        q, k, v = d["q"], d["k"], d["v"]
        ks = k - k.mean(dim=-2, keepdim=True)                      # api.py:184
        out[f"{tag}_q"], out[f"{tag}_k"], out[f"{tag}_v"] = bits(q), bits(k), bits(v)
        out[f"{tag}_ks"] = bits(ks)
        out[f"{tag}_ks_fq"] = bits(rtb(ks))
        out[f"{tag}_v_fq"] = bits(rttb(v))
        sd = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float())
        out[f"{tag}_sdpa"] = sd.numpy()
    # ---- K-packing preprocessing (api.py:112-205), executed unchanged
    import einops
    from typing import Tuple

    def group_mean(q):                     # stands in for triton_group_mean (api.py:26-72): fp32 mean per 128 tokens
        B, H, L, D = q.shape
        g = q.float().reshape(B, H, L // 128, 128, D)
        mean = g.sum(dim=-2) / 128
        return (g - mean.unsqueeze(-2)).to(q.dtype).reshape(B, H, L, D), mean.to(q.dtype)

    (pre,) = lift(ref / "sageattn4" / "api.py", ["preprocess_qkv"],
                  {"E": einops, "F": torch.nn.functional, "Tuple": Tuple, "round_to_blockscaled_fp4": rtb,
                   "round_to_token_blockscaled_fp4": rttb, "triton_group_mean": group_mean})
    pk = {}
    g2 = torch.Generator().manual_seed(7)
    qs = torch.randn(1, 2, 70, 64, generator=g2).to(torch.bfloat16)
    ks_ = (torch.randn(1, 2, 100, 64, generator=g2) + 1.5 * torch.randn(1, 2, 1, 64, generator=g2)).to(torch.bfloat16)
    vs = torch.randn(1, 2, 100, 64, generator=g2).to(torch.bfloat16)
    d128 = torch.load(ref / "tests" / "fixtures" / "llama3p1_8b_instruct_l16_h15_s128_qkv.pt", map_location="cpu")
    for tag, (q, k, v) in {"rand": (qs, ks_, vs), "s128": (d128["q"], d128["k"], d128["v"])}.items():
        qp, kp, vp, ds, lam = pre(q.clone(), k.clone(), v.clone(), True, 16, None)
        pk[f"{tag}_q"], pk[f"{tag}_k"], pk[f"{tag}_v"] = bits(q), bits(k), bits(v)
        pk[f"{tag}_kp"], pk[f"{tag}_vp"] = bits(kp), bits(vp)
        pk[f"{tag}_lam"], pk[f"{tag}_ds"] = lam.float().numpy(), ds.float().numpy()
        # the other kernel variant: whole-sequence Q mean and the split-first V layout (v_trick defaults to True)
        qp0, kp0, vp0, ds0, lam0 = pre(q.clone(), k.clone(), v.clone(), False, 16, None)
        pk[f"{tag}_qs0"], pk[f"{tag}_vp0"], pk[f"{tag}_ds0"] = bits(qp0), bits(vp0), ds0.float().numpy()
        assert torch.equal(kp0, kp) and torch.equal(lam0, lam)      # the K side does not depend on the variant
    np.savez_compressed(HERE / "pack_emulation.npz", **pk)
    print("pack_emulation.npz", {k_: v_.shape for k_, v_ in pk.items()})
    np.savez_compressed(HERE / "llama_fixture_qkv.npz", **out)
    print("llama_fixture_qkv.npz", {k_: v_.shape for k_, v_ in out.items()})


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")
