"""GPU parity of the split-KV decode kernel (Sq <= 64) against the oracle, against the
forward kernel, and across split counts."""
import pytest
import torch

from _util import DTYPES, lse_err, max_abs, qkv
from oracle.attention_oracle import flax_attention_oracle, flax_attention_oracle_chunked

pytestmark = pytest.mark.gpu


def _decode(q, k, v, score_mod, mask_mod, splits=0, path="decode"):
    import flaxattention_b200 as fa

    B, Hq, Sq, _ = q.shape
    Skv = k.shape[2]
    bm = fa.create_block_mask(mask_mod, B, Hq, Sq, Skv) if mask_mod is not None else None
    opts = {"path": path}
    if splits:
        opts["num_splits"] = splits
    out, lse = fa.flax_attention(q.cuda(), k.cuda(), v.cuda(), score_mod=score_mod, block_mask=bm,
                                 enable_gqa=q.shape[1] != k.shape[1], return_lse=True, kernel_options=opts)
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu()


def _mods(Hq, Sq, Skv, mask):
    from flaxattention_b200.masks import causal_mask, generate_causal_offset, generate_sliding_window
    from flaxattention_b200.mods import generate_alibi_bias

    m = {None: None, "offset": generate_causal_offset(Skv - Sq), "literal": causal_mask,
         "window": generate_sliding_window(1000)}[mask]
    return generate_alibi_bias(Hq), m


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("Sq", [1, 7, 16, 33, 64])
@pytest.mark.parametrize("splits", [1, 3, 0])
def test_decode_matches_oracle(Sq, dt, splits):
    B, Hq, Hkv, Skv, D = 2, 4, 4, 2048, 64
    s, m = _mods(Hq, Sq, Skv, "offset")
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, dtype=DTYPES[dt])
    out, lse = _decode(q, k, v, s, m, splits)
    ref, ref_lse = flax_attention_oracle(q, k, v, s, m)
    assert max_abs(out, ref) <= 2e-2
    err, same = lse_err(lse, ref_lse)
    assert same and err <= 2e-2 * max(1.0, ref_lse.abs().max().item())


@pytest.mark.parametrize("case", [
    # B, Hq, Hkv, Sq, Skv, D, mask
    (1, 2, 2, 1, 777, 64, None),          # ragged kv, no mask
    (1, 8, 2, 16, 1500, 128, "offset"),   # GQA, D=128, ragged
    (2, 2, 2, 64, 4096, 64, "literal"),   # the reference's causal_mask taken literally: few visible keys
    (1, 2, 2, 4, 8192, 32, "window"),     # everything masked except a window that the rows never reach
], ids=str)
def test_decode_variants(case):
    B, Hq, Hkv, Sq, Skv, D, mask = case
    s, m = _mods(Hq, Sq, Skv, mask)
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, dtype=torch.float16)
    out, lse = _decode(q, k, v, s, m, 0)
    ref, ref_lse = flax_attention_oracle(q, k, v, s, m)
    assert max_abs(out, ref) <= 2e-2
    err, same = lse_err(lse, ref_lse)
    assert same and err <= 2e-2 * max(1.0, ref_lse[torch.isfinite(ref_lse)].abs().max().item())
    out_f, lse_f = _decode(q, k, v, s, m, 0, path="fwd")
    assert max_abs(out, out_f) <= 4e-3


def test_decode_benchmark_shape():
    """B32 H8 Skv16384 D64 fp16, offset-causal + ALiBi: heads 0..1 of batch 0 against the
    oracle; all rows against a run with a different split count (the result may not depend
    on how the key range is cut)."""
    B, Hq, Skv, D = 32, 8, 16384, 64
    for Sq in (1, 16, 32, 64):
        s, m = _mods(Hq, Sq, Skv, "offset")
        q, k, v = qkv(B, Hq, Hq, Sq, Skv, D, dtype=torch.float16)
        out, lse = _decode(q, k, v, s, m, 0)
        ref, ref_lse = flax_attention_oracle_chunked(q[:1, :2], k[:1, :2], v[:1, :2], s, m, chunk_bh=1)
        assert max_abs(out[:1, :2], ref) <= 2e-2
        assert max_abs(lse[:1, :2], ref_lse) <= 2e-2 * max(1.0, ref_lse.abs().max().item())
        out2, lse2 = _decode(q, k, v, s, m, 12 if Sq > 32 else 5)
        assert max_abs(out, out2) <= 2e-3 and max_abs(lse, lse2) <= 1e-3 * max(1.0, lse.abs().max().item())


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("Sq,splits", [(2, 4), (5, 0), (16, 8), (17, 4), (24, 0), (32, 8), (33, 4), (48, 8), (64, 12), (64, 3), (40, 0), (64, 24)])
def test_tcgen05_decode_and_general_decode_agree_with_the_oracle(Sq, splits, dt):
    """2..64 query rows with a split count that is a multiple of four run on the split-KV variant
    of the tcgen05 kernel (four partial results per CTA: two warpgroups x two column halves), any
    other count or the `general` option on the general decode kernel: both within tolerance of the
    oracle and close to each other, and the status word of the tcgen05 kernel (bounded waits)
    stays 0."""
    import flaxattention_b200 as fa

    B, Hq, Hkv, Skv, D = 2, 4, 4, 3000, 64      # ragged last tile, 24 kv tiles
    s, m = _mods(Hq, Sq, Skv, "offset")
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, dtype=DTYPES[dt])
    ref, ref_lse = flax_attention_oracle(q, k, v, s, m)
    bm = fa.create_block_mask(m, B, Hq, Sq, Skv)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    outs = []
    for opts in ({"path": "decode", "status": status}, {"path": "decode", "kernels": "general"}):
        if splits:
            opts["num_splits"] = splits
        out, lse = fa.flax_attention(q.cuda(), k.cuda(), v.cuda(), score_mod=s, block_mask=bm, return_lse=True,
                                     kernel_options=opts)
        torch.cuda.synchronize()
        assert max_abs(out.cpu(), ref) <= 2e-2
        err, same = lse_err(lse.cpu(), ref_lse)
        assert same and err <= 2e-2 * max(1.0, ref_lse.abs().max().item())
        outs.append(out.cpu())
    assert int(status.item()) == 0
    assert max_abs(outs[0], outs[1]) <= (8e-3 if dt == "f16" else 3.2e-2)


@pytest.mark.parametrize("Hq,Hkv,Sq,dt", [(8, 2, 1, "f16"), (8, 2, 4, "bf16"), (8, 1, 8, "f16"), (4, 2, 16, "f16"),
                                          (16, 4, 16, "bf16")])
def test_grouped_query_decode_packs_the_heads_of_a_group(Hq, Hkv, Sq, dt):
    """GQA decode with tables that do not depend on the head (built with H = 1): the G query heads
    of a kv head share one tile and K / V are read once.  ALiBi depends on the head, so every
    packed row must see its own head index.  Same problem with per-head tables (no packing) and
    through the forward kernel: all within tolerance of the oracle."""
    import ctypes as C

    import flaxattention_b200 as fa
    from flaxattention_b200 import _cabi
    from flaxattention_b200 import attention as A

    B, Skv, D = 2, 3000, 64
    s, m = _mods(Hq, Sq, Skv, "offset")
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, dtype=DTYPES[dt])
    ref, ref_lse = flax_attention_oracle(q, k, v, s, m)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    outs = {}
    for name, heads in (("broadcast", 1), ("per_head", Hq)):
        bm = fa.create_block_mask(m, B, heads, Sq, Skv)
        call = A._Call(qc, kc, vc, s, m, bm, D ** -0.5, "bhsd", 0, 0, None)
        packs = _cabi.lib().fa_decode_packs_heads(C.byref(call.params(qc, kc, vc, qc, None)))
        assert packs == (1 if (name == "broadcast" and (Hq // Hkv) * Sq <= 64) else 0)
        for splits in (0, 1, 3):
            opts = {"path": "decode"}
            if splits:
                opts["num_splits"] = splits
            out, lse = fa.flax_attention(qc, kc, vc, score_mod=s, block_mask=bm, enable_gqa=True, return_lse=True,
                                         kernel_options=opts)
            torch.cuda.synchronize()
            assert max_abs(out.cpu(), ref) <= 2e-2, (name, splits)
            err, same = lse_err(lse.cpu(), ref_lse)
            assert same and err <= 2e-2 * max(1.0, ref_lse.abs().max().item()), (name, splits)
            outs[(name, splits)] = out.cpu()
    assert max_abs(outs[("broadcast", 0)], outs[("per_head", 0)]) <= (4e-3 if dt == "f16" else 3.2e-2)
    fa.check_status()


def test_grouped_query_decode_without_tables_and_sequence_major_layout():
    """No BlockMask at all (packing applies) and [B, L, H, N] inputs: rows of a packed tile come
    from different heads, i.e. from addresses a head stride apart."""
    import flaxattention_b200 as fa
    from flaxattention_b200.mods import generate_alibi_bias

    B, Hq, Hkv, Sq, Skv, D = 2, 8, 2, 3, 1111, 64
    alibi = generate_alibi_bias(Hq)
    q, k, v = qkv(B, Hq, Hkv, Sq, Skv, D, dtype=torch.float16)
    ref, _ = flax_attention_oracle(q, k, v, alibi, None)
    o1 = fa.flax_attention(q.cuda(), k.cuda(), v.cuda(), score_mod=alibi, enable_gqa=True)
    o2 = fa.flax_attention_pallas(q.transpose(1, 2).contiguous().cuda(), k.transpose(1, 2).contiguous().cuda(),
                                  v.transpose(1, 2).contiguous().cuda(), score_mod=alibi, enable_gqa=True, bhln=False)
    torch.cuda.synchronize()
    assert max_abs(o1.cpu(), ref) <= 2e-2
    assert max_abs(o2.cpu().transpose(1, 2), ref) <= 2e-2
