"""The batch x heads partition on real devices: every rank's shard runs on its own GPU with the
global offsets and the gathered result equals the single-GPU one bit for bit (there is no
data-path collective; the gather here only assembles the check).  Needs two visible GPUs."""
import pytest
import torch

from _util import normal, rel_err

pytestmark = pytest.mark.gpu


def _need_two():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


@pytest.mark.parametrize("B,Hq,Hkv,S,D,dt,world", [
    (2, 8, 8, 512, 64, torch.float16, 2),     # 2 x 1 mesh
    (1, 8, 4, 384, 128, torch.bfloat16, 2),   # 1 x 2 mesh: the second rank starts at head 4 (GQA: kv head 2)
    (2, 4, 4, 256, 64, torch.bfloat16, 4),    # 2 x 2 mesh on two devices (ranks alternate)
])
def test_shards_on_two_devices_reproduce_the_single_device_result(B, Hq, Hkv, S, D, dt, world):
    _need_two()
    import flaxattention_b200 as fa
    from cases import head_dependent
    from flaxattention_b200.mods import generate_alibi_bias
    from flaxattention_b200.sharding import shard_for

    alibi = generate_alibi_bias(Hq)
    q, k, v = normal(1, (B, Hq, S, D), dt), normal(0, (B, Hkv, S, D), dt), normal(2, (B, Hkv, S, D), dt)
    dout = normal(7, (B, Hq, S, D), dt)

    def run(dev, qs, ks, vs, ds, bm, b_off, h_off):
        with torch.cuda.device(dev):
            qc, kc, vc = (t.to(dev).requires_grad_(True) for t in (qs, ks, vs))
            out, lse = fa.flax_attention(qc, kc, vc, score_mod=alibi, block_mask=bm, enable_gqa=Hq != Hkv,
                                         return_lse=True, b_offset=b_off, h_offset=h_off)
            out.backward(ds.to(dev))
            torch.cuda.synchronize(dev)
            return [t.detach().cpu() for t in (out, lse, qc.grad, kc.grad, vc.grad)]

    d0 = torch.device("cuda", 0)
    with torch.cuda.device(d0):
        bm_global = fa.create_block_mask(head_dependent, B, Hq, S, S, device=d0)
    ref = run(d0, q, k, v, dout, bm_global, 0, 0)
    got = [torch.zeros_like(t) for t in ref]
    for rank in range(world):
        sh = shard_for(rank, world, B, Hq, Hkv)
        dev = torch.device("cuda", rank % 2)
        with torch.cuda.device(dev):
            # every rank builds the tables of its own shard, on its own device, from the global indices
            bm = fa.create_block_mask(head_dependent, sh.b.stop - sh.b.start, sh.hq.stop - sh.hq.start, S, S,
                                      device=dev, b_offset=sh.b_offset, h_offset=sh.h_offset)
        part = run(dev, q[sh.b, sh.hq], k[sh.b, sh.hkv], v[sh.b, sh.hkv], dout[sh.b, sh.hq], bm, sh.b_offset, sh.h_offset)
        got[0][sh.b, sh.hq], got[1][sh.b, sh.hq], got[2][sh.b, sh.hq] = part[0], part[1], part[2]
        got[3][sh.b, sh.hkv], got[4][sh.b, sh.hkv] = part[3], part[4]
    fa.check_status()
    assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1])
    assert torch.equal(got[3], ref[3]) and torch.equal(got[4], ref[4])
    assert rel_err(got[2], ref[2]) <= 1e-3  # dQ: fp32 reduce-adds in an order that is not fixed
