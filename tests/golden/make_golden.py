"""Generates the golden vectors in this directory.

The reference (zinccat/flaxattention) needs JAX, which is not installed where this was run,
so the vectors come from the oracle its own test-suite uses: eager
``torch.nn.attention.flex_attention`` on CPU (tests/attention_test.py:14-63) and, for the
block tables, ``torch.nn.attention.flex_attention.create_block_mask``, the upstream code the
reference's blockmask.py transcribes.  Gradients come from
``torch.nn.functional.scaled_dot_product_attention`` (no mods), as flex_attention has no CPU
backward.  Inputs are regenerated from seeds by tests/_util.py, so only outputs are stored.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys
import warnings

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from _util import qkv  # noqa: E402
from torch.nn.attention.flex_attention import create_block_mask, flex_attention  # noqa: E402

warnings.filterwarnings("ignore")
HERE = os.path.dirname(os.path.abspath(__file__))


def alibi(H):
    def f(score, b, h, q, kv):
        return score + (q - kv) * torch.exp2(-((h + 1) * 8.0 / H))
    return f


def checkerboard(score, b, h, q, kv):
    score = torch.where((kv - q) % 2 == 0, score * 0.5, score)
    score = torch.where((kv - q) % 2 == 1, score * 2.0, score)
    return score


def causal(b, h, q, kv):
    return q >= kv


def sink(window, sink_size):
    def f(b, h, q, kv):
        return ((kv <= sink_size) | (q - kv <= window)) & (q >= kv)
    return f


def window(w):
    def f(b, h, q, kv):
        return (q - kv <= w) & (q >= kv)
    return f


def causal_offset(off):
    def f(b, h, q, kv):
        return q + off >= kv
    return f


def head_dependent(b, h, q, kv):
    return kv <= q + 64 * h + 32 * b


def attn(name, B, Hq, Hkv, Sq, Skv, D, score_mod=None, mask=None, row_stride=1):
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D)
    bm = create_block_mask(mask, B, Hq, Sq, Skv, device="cpu") if mask is not None else None
    out, lse = flex_attention(q, k, v, score_mod=score_mod, block_mask=bm, enable_gqa=Hq != Hkv, return_lse=True)
    return {f"{name}.out": out[:, :, ::row_stride].numpy(), f"{name}.lse": lse.numpy(),
            f"{name}.shape": np.array([B, Hq, Hkv, Sq, Skv, D, row_stride])}


def tables(name, mask, B, H, Q, KV, bs=128):
    bm = create_block_mask(mask, B, H, Q, KV, device="cpu", BLOCK_SIZE=bs)
    return {f"{name}.{k}": getattr(bm, k).numpy().astype(np.int32)
            for k in ("kv_num_blocks", "kv_indices", "full_kv_num_blocks", "full_kv_indices",
                      "q_num_blocks", "q_indices", "full_q_num_blocks", "full_q_indices")}


def sdpa_grads(name, B, H, Sq, Skv, D):
    q, k, v = qkv(B, H, H, Sq, Skv, D)
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    with torch.nn.attention.sdpa_kernel(torch.nn.attention.SDPBackend.MATH):
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v)
    out.sum().backward()
    return {f"{name}.out": out.detach().numpy(), f"{name}.dq": q.grad.numpy(), f"{name}.dk": k.grad.numpy(),
            f"{name}.dv": v.grad.numpy(), f"{name}.shape": np.array([B, H, H, Sq, Skv, D, 1])}


def main():
    a = {}
    # the reference's own test shapes (tests/attention_test.py: B4 H8 S64 D32 fp32)
    a.update(attn("nomod", 4, 8, 8, 64, 64, 32))
    a.update(attn("decode_alibi", 4, 8, 8, 1, 64, 32, score_mod=alibi(8)))
    a.update(attn("gqa", 2, 8, 2, 64, 64, 32))
    a.update(attn("checkerboard", 2, 4, 4, 64, 96, 32, score_mod=checkerboard))
    # the CPU-runnable benchmark configuration: B2 H4 S256 D64, causal block mask + ALiBi
    a.update(attn("cfg1", 2, 4, 4, 256, 256, 64, score_mod=alibi(4), mask=causal, row_stride=4))
    a.update(attn("sink_ragged", 1, 2, 2, 200, 333, 32, mask=sink(40, 4), row_stride=2))
    a.update(sdpa_grads("grads_nomod", 2, 4, 64, 64, 32))
    a.update(sdpa_grads("grads_decode", 2, 4, 1, 64, 32))
    np.savez_compressed(os.path.join(HERE, "attention_golden.npz"), **a)

    t = {}
    t.update(tables("causal_256", causal, 2, 4, 256, 256))
    t.update(tables("causal_2048", causal, 1, 1, 2048, 2048))
    t.update(tables("sink_8192", sink(1024, 4), 1, 1, 8192, 8192))
    t.update(tables("window_2048_64", window(256), 1, 2, 2048, 2048, 64))
    # Q_LEN < 128 is left out on purpose: the reference then sets Q_BLOCK_SIZE = Q_LEN
    # (flaxattention/core/blockmask.py:440-441) while current torch pads the query to a whole
    # block, so torch is no checker for the decode-shaped grids.  Lengths that are not a
    # multiple of the block are left out as well: the reference evaluates mask_mod on the
    # padded positions (:443-444, :303-322), current torch treats them as masked.
    t.update(tables("head_dependent", head_dependent, 2, 3, 512, 512))
    t.update(tables("all_masked", lambda b, h, q, kv: (q < 0) & (kv < 0), 1, 1, 64, 64))
    np.savez_compressed(os.path.join(HERE, "blockmask_golden.npz"), **t)
    for f in ("attention_golden.npz", "blockmask_golden.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")


if __name__ == "__main__":
    main()
