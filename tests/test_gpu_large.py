"""The one-GPU dMoE-XL shape (BASELINE.json configs[4] on a single device): 64 experts, h = 4096,
f = 14336, 131072 tokens with top-2 routing -> ~266 k padded rows, ~236 k nonzero blocks (7.7 GB of
hidden activations).  The reference's kernels cannot run it (their int32 element offsets overflow
past 2^31 elements of `data`); here the blocks are addressed by TMA row coordinates.  Checked per
expert, on a sample of experts, against dense products of the same operands."""
import pytest
import torch

from tests.parity import assert_product_close

pytestmark = pytest.mark.gpu


def test_dmoe_xl_single_gpu_forward():
    import stk_b200 as stk
    from stk_b200 import dmoe
    from stk_b200.backend import lib
    dev = torch.device("cuda", 0)
    free, _ = torch.cuda.mem_get_info(dev)
    if free < 60 * 2**30:
        pytest.skip("needs ~35 GB of device memory")
    T, h, f, E, dtype = 131072, 4096, 14336, 64, torch.bfloat16
    g = torch.Generator(device=dev).manual_seed(0)
    logits = torch.randn(T, E, generator=g, device=dev)
    probs, ids = torch.topk(torch.softmax(logits, -1), 2, dim=-1)
    ids = ids.to(torch.int32)
    del logits
    index, position, padded, bin_rows, total = dmoe.route_topk(ids, E)
    topo = dmoe.topology_from_bins(bin_rows, total // 128, f, dtype, dev, materialize=False)
    nnz = topo.data.shape[0]
    assert nnz * 128 * 128 > 2**31                       # the regime the reference cannot address
    tokens = torch.empty(T, h, dtype=dtype, device=dev).normal_(0, 0.02, generator=g)
    x = dmoe.permute_tokens(tokens, index, total, top_k=2)
    sample = torch.randint(0, 2 * T, (4096,), generator=g, device=dev)
    assert torch.equal(x[position[sample].long()], tokens[sample // 2])     # every slot holds its token's row
    w1 = torch.empty(h, E * f, dtype=dtype, device=dev).normal_(0, 0.02, generator=g)
    w2 = torch.empty(E * f, h, dtype=dtype, device=dev).normal_(0, 0.02, generator=g)
    with torch.no_grad():
        hid = stk.ops.sdd(x, w1, topo)
        y = stk.ops.dsd(hid, w2)
        rows = (padded // 128).tolist()
        starts = [0]
        for nr in rows:
            starts.append(starts[-1] + nr)
        cpb = f // 128
        for e in (0, 31, 63):                            # first, middle and last expert (last blocks of data)
            r0, nr = starts[e], rows[e]
            assert nr > 0
            sl = slice(r0 * 128, (r0 + nr) * 128)
            he = hid.data[r0 * cpb:(r0 + nr) * cpb].view(nr, cpb, 128, 128).permute(0, 2, 1, 3).reshape(nr * 128, f)
            assert_product_close(he, x[sl].float() @ w1[:, e * f:(e + 1) * f].float(), f"sdd expert {e}")
            assert_product_close(y[sl], he.float() @ w2[e * f:(e + 1) * f].float(), f"dsd expert {e}")
        # the weighted top-2 combine at full size, on a sample of tokens
        out = dmoe.combine_tokens(y, position, probs, T, 2)
        t = torch.randint(0, T, (256,), generator=g, device=dev)
        pos = position.view(T, 2)[t].long()
        expect = (y[pos[:, 0]].float() * probs[t, 0:1] + y[pos[:, 1]].float() * probs[t, 1:2])
        assert_product_close(out[t], expect, "top-2 combine")
    assert lib.device_status() == 0
    del hid, y, x, w1, w2, topo, out, tokens
    torch.cuda.empty_cache()
