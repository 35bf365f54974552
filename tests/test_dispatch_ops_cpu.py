"""The two opaque dispatch ops and the registry behind them, on CPU with stand-in methods - the
contracts the reference pins in tests/test_layer_registry.py:84-350: schema and fake kernels pass
torch.library.opcheck, a compiled caller records exactly ONE node per dispatch with the layer id as
a constant, the padded routes (expert id -1) reach the method untouched (the routing launch drops
them on the device, no elementwise pass and no host read in the op), no prismaquant op is tagged
unsafe for CUDA graphs, and every op has a fake kernel."""
import gc

import pytest
import torch

from gridbook_b200 import ops


class _Layer(torch.nn.Module):
    _cb_N = 5


class _LinearMethod:
    def __init__(self):
        self.seen = []

    def _apply_inline(self, layer, x, bias=None):
        self.seen.append(tuple(x.shape))
        return torch.zeros((*x.shape[:-1], layer._cb_N), dtype=x.dtype, device=x.device)


class _MoEMethod:
    def __init__(self):
        self.seen = []

    def _apply_inline(self, layer, x, topk_weights, topk_ids):
        self.seen.append((topk_weights.clone(), topk_ids.clone()))
        return torch.zeros_like(x)


def test_linear_dispatch_schema_fake_and_output_contract():
    method, layer = _LinearMethod(), _Layer()
    lid = ops.register_cb_layer(method, layer)
    x = torch.ones((2, 3, 7))
    out = ops.cb_linear_forward(x, lid)
    assert out.shape == (2, 3, layer._cb_N) and out.dtype == x.dtype
    torch.library.opcheck(ops.cb_linear_forward, (x, lid))
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode() as mode:
        fake = ops.cb_linear_forward(mode.from_tensor(x), lid)
    assert fake.shape == (2, 3, layer._cb_N) and fake.dtype == x.dtype


def test_moe_dispatch_schema_fake_and_output_contract():
    method, layer = _MoEMethod(), _Layer()
    lid = ops.register_cb_layer(method, layer)
    x, w = torch.ones((3, 7)), torch.ones((3, 2))
    ids = torch.zeros((3, 2), dtype=torch.int64)
    torch.library.opcheck(ops.cb_moe_forward, (x, w, ids, lid))
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode() as mode:
        fake = ops.cb_moe_forward(mode.from_tensor(x), mode.from_tensor(w), mode.from_tensor(ids), lid)
    assert fake.shape == x.shape and fake.dtype == x.dtype


def test_compiled_caller_records_one_opaque_node_per_dispatch():
    traced = []
    method, layer = _MoEMethod(), _Layer()
    lid = ops.register_cb_layer(method, layer)

    def backend(graph, example_inputs):
        traced.append(graph)
        return graph.forward

    def forward(x, w, ids):
        return ops.cb_moe_forward(x, w, ids, lid)

    compiled = torch.compile(forward, backend=backend, fullgraph=True)
    x = torch.ones((4, 7))
    w = torch.tensor([[0.25, 0.75], [0.5, 0.5], [1.0, 0.0], [0.3, 0.7]])
    ids = torch.tensor([[0, -1], [1, 2], [-1, -1], [3, 0]])
    out = compiled(x, w, ids)
    assert torch.equal(out, torch.zeros_like(x))
    assert len(traced) == 1
    nodes = [n for n in traced[0].graph.nodes if n.op == "call_function"]
    assert len(nodes) == 1 and "cb_moe_forward" in str(nodes[0].target)
    assert nodes[0].args[-1] == lid                     # the layer id is a constant of the graph
    # the method sees the routing exactly as the engine wrote it: sentinel ids are dropped by the
    # routing launch on the device, not rewritten by an elementwise pass in front of it
    assert len(method.seen) == 1
    seen_w, seen_ids = method.seen[0]
    assert torch.equal(seen_ids, ids) and torch.equal(seen_w, w)


def test_linear_dispatch_compiles_with_a_static_layer_id():
    method, layer = _LinearMethod(), _Layer()
    lid = ops.register_cb_layer(method, layer)

    def forward(x):
        return ops.cb_linear_forward(x, lid) + 1

    compiled = torch.compile(forward, backend="eager", fullgraph=True)
    out = compiled(torch.ones((2, 7)))
    assert out.shape == (2, layer._cb_N) and torch.equal(out, torch.ones_like(out))
    assert method.seen == [(2, 7)]


def test_padding_sentinel_helper_matches_the_reference_substitution():
    """The helper kept for callers that want the reference's (expert 0, weight 0) substitution
    (gridbook/ops.py:764-784): only the sentinel moves, and nothing is read on the host."""
    w = torch.tensor([[0.25, 0.75], [0.5, 0.5]])
    ids = torch.tensor([[0, -1], [-1, 2]])
    w2, ids2 = ops._neutralize_moe_padding_sentinel(w, ids)
    assert torch.equal(ids2, torch.tensor([[0, 0], [0, 2]]))
    assert torch.equal(w2, torch.tensor([[0.25, 0.0], [0.0, 0.5]]))
    assert torch.equal(ids, torch.tensor([[0, -1], [-1, 2]]))       # inputs untouched


def test_stale_and_expired_ids_fail_loudly():
    method, layer = _LinearMethod(), _Layer()
    lid = ops.register_cb_layer(method, layer)
    x = torch.ones((1, 7))
    del layer
    gc.collect()
    with pytest.raises(RuntimeError, match="stale or unknown|expired"):
        ops.cb_linear_forward(x, lid)
    with pytest.raises(RuntimeError, match="stale or unknown"):
        ops.cb_linear_forward(x, 10 ** 9)


def _prismaquant_ops():
    names = [n for n in dir(torch.ops.prismaquant) if not n.startswith("_")]
    found = []
    for n in names:
        packet = getattr(torch.ops.prismaquant, n)
        if not hasattr(packet, "overloads"):
            continue          # a plain attribute of the namespace, not an op
        for overload in packet.overloads():
            found.append((n, getattr(packet, overload)))
    return found


def test_no_prismaquant_op_claims_cudagraph_unsafe_and_every_op_has_a_fake():
    found = _prismaquant_ops()
    assert len(found) >= 20, f"only {len(found)} prismaquant ops are registered"
    for name, op in found:
        assert torch.Tag.cudagraph_unsafe not in op.tags, f"{name} is tagged cudagraph_unsafe"
        # a fake (meta) kernel is what lets the compiler trace through the op without running it
        assert torch._C._dispatch_has_kernel_for_dispatch_key(op.name(), "Meta") or \
            torch._C._dispatch_has_kernel_for_dispatch_key(op.name(), "CompositeExplicitAutograd") or \
            _has_fake(op), f"{name} has no fake kernel"


def _has_fake(op) -> bool:
    try:
        from torch._library.simple_registry import singleton
        return singleton.find(op.name()).fake_impl.kernel is not None
    except Exception:
        return False


def test_the_reference_op_names_on_the_path_exist():
    """Names a caller of the reference's ops layer binds (gridbook/ops.py:52-428,731-798)."""
    want = ["cb_gemv_fp8", "cb_gemv_fp4_v2", "cb_expand_fp8", "cb_expand_fp4_v2", "fp8_act_qdq", "fp4_act_qdq",
            "cb_moe_gemv_fp4_v2", "cb_moe_gemv_v2", "cb_moe_gemv_fp8", "cb_moe_gemv_fp8_v2", "cb_moe_combine",
            "cb_bf16_grouped_mm", "cb_bf16_grouped_mm_out", "cb_moe_persistent_b_prefill",
            "cb_moe_persistent_b_prefill_d2r", "cb_moe_persistent_b_prefill_fp8", "cb_moe_persistent_b_decode",
            "cb_moe_persistent_b_decode_fp8", "cb_linear_forward", "cb_moe_forward"]
    for n in want:
        assert hasattr(torch.ops.prismaquant, n), n
