"""Whole-layer CUDA-graph capture (the engine's FULL decode graphs, docs/KERNELS.md:1018-1071 of the
reference): a decoder block's codebook linears and its routed layer, driven through the plugin
methods, are captured at every decode size AND at prefill sizes - none of the routes reads a
device value on the host - and a replay on new inputs returns what eager execution returns, bit
for bit (capture on == capture off)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def block():
    """q, kv, o, gate_up, down (small shapes with the stack's proportions) + one routed layer."""
    from gridbook_b200 import _native, synth
    from gridbook_b200.formats import NVFP4_LITERAL
    from gridbook_b200.linear import CBLinear
    from gridbook_b200.moe import CBMoE
    _native.prepare(0)
    dev = torch.device("cuda:0")
    fmt = NVFP4_LITERAL
    hidden, inter = 1024, 2048
    gen = torch.Generator(device=dev).manual_seed(3)
    shapes = {"q": ([768], hidden), "kv": ([128, 128], hidden), "o": ([hidden], 768),
              "gate_up": ([inter, inter], hidden), "down": ([hidden], inter)}
    lins = {}
    for i, (name, (parts, K)) in enumerate(shapes.items()):
        lin = CBLinear(fmt, K, parts, [synth.codebook_tables(fmt, i)], global_scale=1.0 / 448.0, prefix=f"blk.{name}")
        lins[name] = lin.load(synth.make_packed_device(fmt, sum(parts), K, gen, dev), None, dev)
    E, topk, minter = 16, 4, 256
    moe = CBMoE(fmt, fmt, E, hidden, minter, synth.codebook_tables(fmt, 7), synth.codebook_tables(fmt, 8))
    moe.load(synth.make_packed_device(fmt, E * 2 * minter, hidden, gen, dev).view(E, 2 * minter, -1),
             synth.make_packed_device(fmt, E * hidden, minter, gen, dev).view(E, hidden, -1), None, None, dev)
    return dev, lins, moe, hidden, inter, E, topk


def _forward(lins, moe, inter, x, tw, ids):
    from gridbook_b200.linear import apply_shared_row
    q, kv = apply_shared_row([lins["q"], lins["kv"]], x)
    a = lins["o"](q)                                     # stands in for attention: shapes only
    h = lins["gate_up"](a)
    y = lins["down"](torch.nn.functional.silu(h[..., :inter]) * h[..., inter:])
    return y + moe(a, tw, ids), kv


@pytest.mark.parametrize("T", [1, 2, 4, 8, 16, 40, 300, 1800])
def test_block_capture_equals_eager(block, T):
    from gridbook_b200 import _native, synth
    dev, lins, moe, hidden, inter, E, topk = block
    ids, tw = synth.make_routing(T, E, topk, seed=T)
    x = synth.bf16_tensor(synth.make_activations(T, hidden, seed=T), dev)
    tw_d, ids_d = torch.from_numpy(tw).to(dev), torch.from_numpy(ids).to(dev)
    _forward(lins, moe, inter, x, tw_d, ids_d)           # warm-up outside the capture
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        out, kv = _forward(lins, moe, inter, x, tw_d, ids_d)
    for seed in (100 + T, 200 + T):                      # two replays on new inputs and new routings
        ids2, tw2 = synth.make_routing(T, E, topk, seed=seed)
        x.copy_(synth.bf16_tensor(synth.make_activations(T, hidden, seed=seed), dev))
        tw_d.copy_(torch.from_numpy(tw2).to(dev))
        ids_d.copy_(torch.from_numpy(ids2).to(dev))
        g.replay()
        torch.cuda.synchronize()
        want, want_kv = _forward(lins, moe, inter, x, tw_d, ids_d)
        torch.cuda.synchronize()
        assert torch.equal(out, want) and torch.equal(kv, want_kv), (T, seed)
    assert _native.device_status(0) == 0
