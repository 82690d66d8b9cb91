"""Generate the golden fixtures in this folder by running the reference's own PyTorch attention.

Run once in a container that has the reference checkout, giving its path:

    python tests/golden/make_golden.py /path/to/HipKittens

It imports ``llama.models.attentions.base.CrossAttention`` / ``SelfAttention`` from the reference's
``training/llama`` tree and evaluates them on seeded bf16-valued inputs, once on fp32 copies (then the
reference computes its softmax in fp32 and its result is the parity target to ~1e-6) and, for the
first case, once natively in bf16 (its stock behaviour; looser agreement, recorded for context).

Each ``case_*.npz`` holds the inputs as raw bf16 bit patterns (uint16), the reference outputs, and the
logsumexp of the reference's own score expression ``einsum(q, k * scale)`` evaluated in fp64 -- the
reference has no CPU path that returns L, so that array pins L's definition, not a reference output.
The GPU box has no reference checkout; tests read only the committed ``.npz`` files.
"""
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, B, N, H, H_KV, D, causal, seed)
CASES = [
    ("c1_b1_n256_h8_kv2_d64_nc", 1, 256, 8, 2, 64, False, 0),
    ("b1_n128_h4_kv2_d64_causal", 1, 128, 4, 2, 64, True, 1),
    ("b2_n128_h2_kv1_d128_causal", 2, 128, 2, 1, 128, True, 2),
    ("b1_n256_h2_kv2_d128_nc", 1, 256, 2, 2, 128, False, 3),
]
# key-padding case: (name, B, N, H, H_KV, D, seed, kv_lens); run through CrossAttention's key_padding_mask
PADDED = ("b3_n256_h4_kv2_d64_keypad", 3, 256, 4, 2, 64, 4, [256, 100, 129])


def reference_root() -> str:
    if len(sys.argv) < 2 or not os.path.isdir(os.path.join(sys.argv[1], "training", "llama")):
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/HipKittens")
    return sys.argv[1]


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    ref_root = reference_root()
    sys.path.insert(0, os.path.join(ref_root, "training", "llama"))
    from llama.models.attentions.base import CrossAttention, SelfAttention  # noqa: E402

    for name, b, n, h, hkv, d, causal, seed in CASES:
        gen = torch.Generator().manual_seed(seed)
        q = torch.randn((b, n, h, d), generator=gen).to(torch.bfloat16)
        k = torch.randn((b, n, hkv, d), generator=gen).to(torch.bfloat16)
        v = torch.randn((b, n, hkv, d), generator=gen).to(torch.bfloat16)
        d_o = torch.randn((b, n, h, d), generator=gen).to(torch.bfloat16)  # drawn last: q, k, v keep their values
        attn = CrossAttention(causal=causal)
        # backward of the reference module: autograd through base.py:78-120 on fp32 leaves
        qf = q.float().requires_grad_(True)
        kvf = torch.stack([k.float(), v.float()], dim=2).requires_grad_(True)
        attn(qf, kvf).backward(d_o.float())
        grads = {"d_o": bf16_bits(d_o), "dq_ref_fp32": qf.grad.numpy().astype(np.float32),
                 "dk_ref_fp32": kvf.grad[:, :, 0].contiguous().numpy().astype(np.float32),
                 "dv_ref_fp32": kvf.grad[:, :, 1].contiguous().numpy().astype(np.float32)}
        with torch.no_grad():
            o32 = attn(q.float(), torch.stack([k.float(), v.float()], dim=2))
            out = {"q": bf16_bits(q), "k": bf16_bits(k), "v": bf16_bits(v),
                   "o_ref_fp32": o32.numpy().astype(np.float32),
                   "shape": np.array([b, n, h, hkv, d, int(causal), seed], dtype=np.int64)}
            out.update(grads)
            if h == hkv:
                # MHA: the SelfAttention module must agree with CrossAttention on the same inputs.
                o_self = SelfAttention(causal=causal)(torch.stack([q.float(), k.float(), v.float()], dim=2))
                assert torch.allclose(o_self, o32, atol=1e-6), "reference modules disagree"
            if name.startswith("c1_"):
                o16 = attn(q, torch.stack([k, v], dim=2))
                out["o_ref_native_bf16"] = bf16_bits(o16)
            # L: logsumexp of the reference's score expression (base.py:96), in fp64.
            g = h // hkv
            kk = k.double().repeat_interleave(g, dim=2)
            scores = torch.einsum("bthd,bshd->bhts", q.double(), kk * (1.0 / math.sqrt(d)))
            if causal:
                mask = torch.triu(torch.ones(n, n, dtype=torch.bool), 1)
                scores = scores.masked_fill(mask, float("-inf"))
            out["lse_def_fp64"] = torch.logsumexp(scores, dim=-1).numpy()  # [B,H,N]
        path = os.path.join(HERE, f"case_{name}.npz")
        np.savez_compressed(path, **out)
        print("wrote", path, os.path.getsize(path), "bytes")

    name, b, n, h, hkv, d, seed, lens = PADDED
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn((b, n, h, d), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, n, hkv, d), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, n, hkv, d), generator=gen).to(torch.bfloat16)
    d_o = torch.randn((b, n, h, d), generator=gen).to(torch.bfloat16)  # drawn last: q, k, v keep their values
    keep = torch.arange(n).view(1, n) < torch.tensor(lens).view(b, 1)  # True = keep (base.py:88-89)
    qf = q.float().requires_grad_(True)
    kvf = torch.stack([k.float(), v.float()], dim=2).requires_grad_(True)
    CrossAttention(causal=False)(qf, kvf, key_padding_mask=keep).backward(d_o.float())
    with torch.no_grad():
        o32 = CrossAttention(causal=False)(q.float(), torch.stack([k.float(), v.float()], dim=2), key_padding_mask=keep)
        kk = k.double().repeat_interleave(h // hkv, dim=2)
        scores = torch.einsum("bthd,bshd->bhts", q.double(), kk * (1.0 / math.sqrt(d)))
        scores = scores.masked_fill(~keep.view(b, 1, 1, n), float("-inf"))
        lse = torch.logsumexp(scores, dim=-1).numpy()
    path = os.path.join(HERE, f"case_{name}.npz")
    np.savez_compressed(path, q=bf16_bits(q), k=bf16_bits(k), v=bf16_bits(v), o_ref_fp32=o32.numpy().astype(np.float32),
                        lse_def_fp64=lse, kv_lens=np.array(lens, dtype=np.int32), d_o=bf16_bits(d_o),
                        dq_ref_fp32=qf.grad.numpy().astype(np.float32),
                        dk_ref_fp32=kvf.grad[:, :, 0].contiguous().numpy().astype(np.float32),
                        dv_ref_fp32=kvf.grad[:, :, 1].contiguous().numpy().astype(np.float32),
                        shape=np.array([b, n, h, hkv, d, 0, seed], dtype=np.int64))
    print("wrote", path, os.path.getsize(path), "bytes")


def rotary_main() -> None:
    """Rotary fixture from the reference harness's own ``get_cos_sin`` / ``get_output``
    (kernels/rotary/test_python.py:36-58). The harness imports its compiled module at the top, so the two functions
    are taken out of its source with ``ast`` and executed on CPU tensors."""
    import ast

    from einops import repeat

    ref_root = reference_root()
    src = open(os.path.join(ref_root, "kernels", "rotary", "test_python.py")).read()
    tree = ast.parse(src)
    wanted = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in ("get_cos_sin", "get_output")]
    assert len(wanted) == 2
    b, h, n, d = 2, 3, 160, 128
    ns = {"torch": torch, "repeat": repeat, "N": n, "D": d}
    exec(compile(ast.Module(body=wanted, type_ignores=[]), "rotary_harness_functions", "exec"), ns)
    gen = torch.Generator().manual_seed(5)
    x = torch.randn((b, h, n, d), generator=gen).to(torch.bfloat16)
    cos_in, sin_in, ro_dim = ns["get_cos_sin"](x, rotary_emb_dim=d)
    out = ns["get_output"](x, cos_in, sin_in, ro_dim)
    path = os.path.join(HERE, "rotary_b2_h3_n160_d128.npz")
    np.savez_compressed(path, x=bf16_bits(x), cos=bf16_bits(cos_in), sin=bf16_bits(sin_in), o_ref=bf16_bits(out),
                        shape=np.array([b, h, n, d, ro_dim], dtype=np.int64))
    print("wrote", path, os.path.getsize(path), "bytes")


def lse_pin_main() -> None:
    """Pin L by the reference code that CONSUMES it: ``simple_flash_backward(Q, K, V, dO, L)`` of the backward
    harness (kernels/attn/gqa_backwards/test_python.py:100-137) recomputes P = exp(Q K^T scale - L) from a saved L
    and derives dQ, dK, dV from that P. The function and its helper ``expand_kv_for_gqa`` (test_python.py:74-80) are
    taken out of the harness source with ``ast`` (the file imports its compiled modules and AITER at the top) and
    run in fp64 on the non-causal fixtures' inputs (the function applies no mask) with the L this repository's
    oracle computes. Stored per case in ``lpin_<case>.npz``:
      lse_fed      the L that was fed in, fp32 [B,H,N] (natural log, scaled logits)
      p_rowsum     row sums of the function's own P: its Delta output for V = 1, dO = 1/D (then O = rowsum(P) in
                   every column and Delta = sum_d dO * O = rowsum(P)); 1 exactly iff L is what the function expects
      dq/dk/dv     its gradients for the fixture's dO, to be compared with the module's autograd gradients that
                   the case_*.npz files already hold
    """
    import ast

    ref_root = reference_root()
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.attn_oracle import attn_fwd_oracle

    src = open(os.path.join(ref_root, "kernels", "attn", "gqa_backwards", "test_python.py")).read()
    tree = ast.parse(src)
    wanted = [n for n in tree.body
              if isinstance(n, ast.FunctionDef) and n.name in ("expand_kv_for_gqa", "simple_flash_backward")]
    assert len(wanted) == 2
    for name, b, n, h, hkv, d, causal, _seed in CASES:
        if causal:
            continue
        z = np.load(os.path.join(HERE, f"case_{name}.npz"))
        unbits = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)  # noqa: E731
        q, k, v, d_o = (unbits(z[key]) for key in ("q", "k", "v", "d_o"))
        _o, lse = attn_fwd_oracle(q, k, v, False)                    # [B,H,1,N] fp32
        lse_bhn = lse[:, :, 0, :].contiguous()
        ns = {"torch": torch, "math": math, "h_q": h, "h_kv": hkv}
        exec(compile(ast.Module(body=wanted, type_ignores=[]), "gqa_backwards_harness_functions", "exec"), ns)
        sfb = ns["simple_flash_backward"]
        to_bhnd = lambda t: t.double().permute(0, 2, 1, 3).contiguous()  # noqa: E731
        qd, kd, vd, dod = to_bhnd(q), to_bhnd(k), to_bhnd(v), to_bhnd(d_o)
        _dq1, _dk1, _dv1, rowsum = sfb(qd, kd, torch.ones_like(vd), torch.full_like(dod, 1.0 / d), lse_bhn.double())
        dq, dk, dv, _delta = sfb(qd, kd, vd, dod, lse_bhn.double())
        path = os.path.join(HERE, f"lpin_{name}.npz")
        np.savez_compressed(path, lse_fed=lse_bhn.numpy(), p_rowsum=rowsum[..., 0].numpy(),
                            dq=dq.permute(0, 2, 1, 3).float().numpy(), dk=dk.permute(0, 2, 1, 3).float().numpy(),
                            dv=dv.permute(0, 2, 1, 3).float().numpy())
        print("wrote", path, os.path.getsize(path), "bytes; max |rowsum(P) - 1| =",
              float((rowsum - 1).abs().max()))


# (name, B, Sq, Sk, H, H_KV, D, causal, seed, kv_lens or None)
CROSS = [
    # a query block shorter than the keys, causal, with key padding: what inference with a cache calls
    # (mha.py:164-168); every row sees at least one key (kept keys >= queries)
    ("b3_q100_k256_h4_kv2_d64_causal_keypad", 3, 100, 256, 4, 2, 64, True, 11, [256, 130, 100]),
    # plain cross attention, neither length a multiple of the tile
    ("b2_q72_k320_h2_kv1_d128_nc", 2, 72, 320, 2, 1, 128, False, 12, None),
    # causal self-attention on a right-padded batch: with 200 kept keys of 256 the reference's mask
    # col > row + 200 - 256 leaves rows 0..55 of that batch element without any key
    ("b2_n256_h2_kv1_d128_causal_keypad", 2, 256, 256, 2, 1, 128, True, 13, [256, 200]),
    # more queries than keys, causal, no padding: the first Sq - Sk rows see nothing
    ("b1_q300_k130_h2_kv2_d64_causal", 1, 300, 130, 2, 2, 64, True, 14, None),
]


def cross_main() -> None:
    """Fixtures for Sq != Sk and for causal together with key padding, through the reference's
    ``CrossAttention(causal=...)(q, kv, key_padding_mask=...)`` (base.py:78-120) on fp32 copies, forward and autograd
    gradients. Where the reference's mask leaves a query row without any key its -10000 fill makes the row attend
    uniformly to masked keys; ``row_valid`` marks the rows that see at least one key, the upstream gradient is zero
    on the other rows (so that they contribute nothing to dK and dV in the reference either), and only valid rows of
    O are to be compared."""
    ref_root = reference_root()
    sys.path.insert(0, os.path.join(ref_root, "training", "llama"))
    from llama.models.attentions.base import CrossAttention  # noqa: E402

    for name, b, sq, sk, h, hkv, d, causal, seed, lens in CROSS:
        gen = torch.Generator().manual_seed(seed)
        q = torch.randn((b, sq, h, d), generator=gen).to(torch.bfloat16)
        k = torch.randn((b, sk, hkv, d), generator=gen).to(torch.bfloat16)
        v = torch.randn((b, sk, hkv, d), generator=gen).to(torch.bfloat16)
        d_o = torch.randn((b, sq, h, d), generator=gen).to(torch.bfloat16)
        kept = torch.tensor(lens if lens is not None else [sk] * b)
        keep = (torch.arange(sk).view(1, sk) < kept.view(b, 1)) if lens is not None else None
        row_valid = (torch.arange(sq).view(1, sq) + (kept.view(b, 1) - sq) >= 0) if causal else torch.ones(b, sq, dtype=torch.bool)
        d_o = d_o * row_valid.view(b, sq, 1, 1).to(torch.bfloat16)
        attn = CrossAttention(causal=causal)
        qf = q.float().requires_grad_(True)
        kvf = torch.stack([k.float(), v.float()], dim=2).requires_grad_(True)
        o32 = attn(qf, kvf, key_padding_mask=keep)
        o32.backward(d_o.float())
        kk = k.double().repeat_interleave(h // hkv, dim=2)
        scores = torch.einsum("bthd,bshd->bhts", q.double(), kk * (1.0 / math.sqrt(d)))
        col = torch.arange(sk).view(1, 1, 1, sk)
        scores = scores.masked_fill(col >= kept.view(b, 1, 1, 1), float("-inf"))
        if causal:
            row = torch.arange(sq).view(1, 1, sq, 1)
            scores = scores.masked_fill(col > row + (kept.view(b, 1, 1, 1) - sq), float("-inf"))
        out = {"q": bf16_bits(q), "k": bf16_bits(k), "v": bf16_bits(v), "d_o": bf16_bits(d_o),
               "o_ref_fp32": o32.detach().numpy().astype(np.float32), "row_valid": row_valid.numpy(),
               "dq_ref_fp32": qf.grad.numpy().astype(np.float32),
               "dk_ref_fp32": kvf.grad[:, :, 0].contiguous().numpy().astype(np.float32),
               "dv_ref_fp32": kvf.grad[:, :, 1].contiguous().numpy().astype(np.float32),
               "lse_def_fp64": torch.logsumexp(scores, dim=-1).numpy(),
               "shape": np.array([b, sq, sk, h, hkv, d, int(causal), seed], dtype=np.int64)}
        if lens is not None:
            out["kv_lens"] = np.array(lens, dtype=np.int32)
        path = os.path.join(HERE, f"cross_{name}.npz")
        np.savez_compressed(path, **out)
        print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
    rotary_main()
    lse_pin_main()
    cross_main()
