"""CPU tests of the graph builder and runtime: construct semantics, naming, structural hash,
forward references, control flow, tree paths, observation, profiling, rendering."""
import os

import pytest
import torch

from flodl_b200 import nn
from flodl_b200.autograd import Variable
from flodl_b200.graph import (ArgmaxSelector, FixedSelector, FlowBuilder, Graph, MergeOp, Reduce, Reshape, SoftmaxRouter,
                              StateAdd, ThresholdHalt, topological_levels)
from flodl_b200.nn.module import Module


def V(t):
    return Variable(t)


class Scale(Module):
    def __init__(self, k):
        self.k = k

    def name(self):
        return "scale"

    def forward(self, x):
        return x.mul_scalar(self.k)


class AddRef(Module):
    """Named-input module: adds the reference called `ctx` to the stream."""

    def name(self):
        return "addref"

    def forward(self, x):
        return x

    def as_named_input(self):
        return self

    def forward_named(self, x, refs):
        return x.add(refs["ctx"])


# ---- builder basics --------------------------------------------------------------------------------
def test_through_chain_and_node_names():
    torch.manual_seed(0)
    g = FlowBuilder.from_(nn.Linear(4, 8)).through(nn.ReLU()).through(nn.Linear(8, 2)).build()
    names = [n for n, _ in g.named_parameters()]
    assert names == ["linear_1/weight", "linear_1/bias", "linear_3/weight", "linear_3/bias"]
    y = g.forward(V(torch.randn(5, 4)))
    assert list(y.t.shape) == [5, 2]


def test_tag_names_parameters_and_is_readable():
    g = (FlowBuilder.from_(nn.Linear(4, 4)).tag("enc").through(nn.Linear(4, 2)).tag("head").build())
    names = [n for n, _ in g.named_parameters()]
    assert names[0] == "enc/weight" and names[2] == "head/weight"
    g.forward(V(torch.randn(3, 4)))
    assert list(g.tagged("enc").t.shape) == [3, 4]
    assert g.tagged("nope") is None


def test_also_is_residual_add():
    g = FlowBuilder.from_(Scale(1.0)).also(Scale(2.0)).build()
    x = torch.randn(3, 4)
    torch.testing.assert_close(g.forward(V(x)).t, 3.0 * x)


def test_split_merge_add_and_mean():
    x = torch.randn(2, 3)
    g = FlowBuilder.from_(Scale(1.0)).split([Scale(1.0), Scale(3.0)]).merge(MergeOp.Add).build()
    torch.testing.assert_close(g.forward(V(x)).t, 4.0 * x)
    g = FlowBuilder.from_(Scale(1.0)).split([Scale(1.0), Scale(3.0)]).merge(MergeOp.Mean).build()
    torch.testing.assert_close(g.forward(V(x)).t, 2.0 * x)


def test_fork_keeps_main_stream():
    g = FlowBuilder.from_(Scale(2.0)).fork(Scale(10.0)).tag("side").through(Scale(3.0)).build()
    x = torch.ones(2, 2)
    torch.testing.assert_close(g.forward(V(x)).t, 6.0 * x)
    torch.testing.assert_close(g.tagged("side").t, 20.0 * x)


def test_using_backward_reference():
    g = (FlowBuilder.from_(Scale(2.0)).tag("ctx").through(Scale(5.0)).through(AddRef()).using(["ctx"]).build())
    x = torch.ones(2, 2)
    torch.testing.assert_close(g.forward(V(x)).t, 12.0 * x)


def test_forward_reference_carries_state_between_calls():
    # `using("ctx")` before `tag("ctx")`: first call sees zeros (nothing yet), later calls the previous value
    g = (FlowBuilder.from_(Scale(1.0)).through(StateAdd()).using(["ctx"]).tag("ctx").build())
    x = torch.ones(1, 2)
    assert g.has_state()
    y1 = g.forward(V(x)).t
    y2 = g.forward(V(x)).t
    y3 = g.forward(V(x)).t
    torch.testing.assert_close(y1, x)
    torch.testing.assert_close(y2, 2 * x)
    torch.testing.assert_close(y3, 3 * x)
    g.reset_state()
    torch.testing.assert_close(g.forward(V(x)).t, x)


def test_multi_input_graph():
    g = (FlowBuilder.from_(Scale(1.0)).input(["b"]).through(AddRef2()).using(["b"]).build())
    a, b = torch.ones(2, 2), torch.full((2, 2), 3.0)
    torch.testing.assert_close(g.forward([V(a), V(b)]).t, a + b)
    with pytest.raises(Exception):
        g.forward([V(a)])


class AddRef2(AddRef):
    def forward_named(self, x, refs):
        return x.add(refs["b"])


def test_errors_surface_at_build():
    with pytest.raises(Exception) as e:
        FlowBuilder.from_(Scale(1.0)).tag("a").through(Scale(1.0)).tag("a").build()
    assert "a" in str(e.value)
    with pytest.raises(Exception):
        FlowBuilder.from_(Scale(1.0)).merge().build()       # merge without split
    with pytest.raises(Exception):
        FlowBuilder.from_(Scale(1.0)).through(AddRef()).using(["missing"]).through(Scale(1.0)).build()


# ---- control flow ----------------------------------------------------------------------------------
def test_loop_for_n():
    g = FlowBuilder.from_(Scale(1.0)).loop_body(Scale(2.0)).for_n(3).build()
    x = torch.ones(2)
    torch.testing.assert_close(g.forward(V(x)).t, 8.0 * x)


def test_loop_until_halts_on_threshold():
    g = FlowBuilder.from_(Scale(1.0)).loop_body(Scale(2.0)).until_cond(ThresholdHalt(10.0), 20).build()
    y = g.forward(V(torch.ones(1))).t
    assert 10.0 < float(y) <= 32.0


def test_switch_selects_one_branch():
    g = FlowBuilder.from_(Scale(1.0)).switch(FixedSelector(1), [Scale(2.0), Scale(5.0)]).build()
    x = torch.ones(2, 2)
    torch.testing.assert_close(g.forward(V(x)).t, 5.0 * x)


def test_gate_mixes_experts_with_router_weights():
    torch.manual_seed(1)
    router = SoftmaxRouter(4, 2)
    g = FlowBuilder.from_(Scale(1.0)).gate(router, [Scale(1.0), Scale(3.0)]).build()
    x = torch.randn(5, 4)
    y = g.forward(V(x)).t
    w = router.forward(V(x)).t
    torch.testing.assert_close(y, x * w[:, :1] + 3.0 * x * w[:, 1:2])
    y.sum().backward()
    assert all(p.t.grad is not None for p in router.parameters())


def test_map_each_and_slices():
    g = FlowBuilder.from_(Scale(1.0)).map(Scale(2.0)).each().build()
    x = torch.randn(3, 4)
    torch.testing.assert_close(g.forward(V(x)).t, 2.0 * x)
    g = FlowBuilder.from_(Scale(1.0)).map(Scale(2.0)).slices(2).build()
    torch.testing.assert_close(g.forward(V(x)).t, 2.0 * x)
    g = FlowBuilder.from_(Scale(1.0)).map(Scale(2.0)).batched().each().build()
    torch.testing.assert_close(g.forward(V(x)).t, 2.0 * x)


def test_reshape_helper():
    g = FlowBuilder.from_(Reshape([-1, 2])).build()
    assert list(g.forward(V(torch.zeros(3, 4))).t.shape) == [6, 2]


# ---- identity ---------------------------------------------------------------------------------------
def _mlp(hidden=8):
    return FlowBuilder.from_(nn.Linear(4, hidden)).tag("a").through(nn.GELU()).through(nn.Linear(hidden, 2)).tag("b").build()


def test_structural_hash_is_stable_and_shape_sensitive():
    h1, h2, h3 = _mlp().structural_hash(), _mlp().structural_hash(), _mlp(16).structural_hash()
    assert len(h1) == 64 and h1 == h2 and h1 != h3
    assert _mlp().short_hash() == h1[:8]
    lab = FlowBuilder.from_(nn.Linear(4, 8)).tag("a").through(nn.GELU()).through(nn.Linear(8, 2)).tag("b").label("enc").build()
    assert lab.structural_hash() == h1          # the label is not part of the hash


def test_topological_levels():
    lv = topological_levels(4, [(0, 1), (0, 2), (1, 3), (2, 3)])
    assert lv == [[0], [1, 2], [3]]
    with pytest.raises(Exception):
        topological_levels(2, [(0, 1), (1, 0)])


def test_parameters_are_deduplicated_for_shared_modules():
    lin = nn.Linear(4, 4)
    g = FlowBuilder.from_(lin).through(nn.ReLU()).through(lin).build()
    assert len(g.parameters()) == 2


# ---- tree -------------------------------------------------------------------------------------------
def _nested():
    enc = FlowBuilder.from_(nn.Linear(4, 4)).tag("proj").through(nn.ReLU()).tag("_hidden").label("encoder").build()
    return FlowBuilder.from_(enc).through(nn.Linear(4, 2)).tag("head").label("model").build()


def test_tree_paths_freeze_and_thaw():
    g = _nested()
    assert "encoder" in g.tree_children()
    assert len(g.parameters_at("encoder")) == 2
    assert len(g.parameters_at("encoder.proj")) == 2
    assert len(g.parameters_at("head")) == 2
    g.freeze("encoder")
    assert g.is_frozen("encoder") and not g.is_frozen("head")
    out = g.forward(V(torch.randn(3, 4)))
    out.t.sum().backward()
    enc_p = g.parameters_at("encoder")
    assert all(p.t.grad is None for p in enc_p)
    assert all(p.t.grad is not None for p in g.parameters_at("head"))
    g.thaw("encoder")
    assert not g.is_frozen("encoder")
    assert len(g.parameters()) == 4            # frozen or not, all are listed


def test_internal_tags_are_not_reachable_across_a_boundary():
    g = _nested()
    with pytest.raises(Exception):
        g.validate_path("encoder._hidden")
    assert g.validate_path("encoder.proj") is not None
    with pytest.raises(Exception):
        g.validate_path("nothing.here")


def test_label_rules():
    child = FlowBuilder.from_(nn.Linear(2, 2)).label("a.b").build()
    with pytest.raises(Exception):                        # dots are path separators
        FlowBuilder.from_(child).build()
    c1 = FlowBuilder.from_(nn.Linear(2, 2)).label("same").build()
    c2 = FlowBuilder.from_(nn.Linear(2, 2)).label("same").build()
    with pytest.raises(Exception):                        # unique per level
        FlowBuilder.from_(c1).through(c2).build()


def test_subgraph_checkpoint_roundtrip(tmp_path):
    g1, g2 = _nested(), _nested()
    path = str(tmp_path / "enc.fdl")
    g1.subgraph("encoder").save_checkpoint(path)
    rep = g2.load_subgraph_checkpoint("encoder", path)
    assert len(rep.loaded) == 2
    for (n1, p1), (n2, p2) in zip(g1.named_parameters_at("encoder"), g2.named_parameters_at("encoder")):
        assert n1 == n2 and torch.equal(p1.t, p2.t)


# ---- observation -----------------------------------------------------------------------------------
class MeanLoss(Module):
    def name(self):
        return "meanloss"

    def forward(self, x):
        return x.mean()


def test_collect_flush_trend():
    g = FlowBuilder.from_(Scale(1.0)).through(MeanLoss()).tag("loss").build()
    for epoch in range(4):
        for b in range(3):
            g.forward(V(torch.full((2, 2), float(10 - 2 * epoch))))
            g.collect(["loss"])
        g.flush(["loss"])
    tr = g.trend("loss")
    assert tr.len() == 4 and tr.values() == [10.0, 8.0, 6.0, 4.0]
    assert abs(tr.slope(0) + 2.0) < 1e-9
    assert tr.improving(0) and not tr.stalled(0, 1e-3)
    assert g.flush_count() == 4
    g.record_scalar("acc", 0.5)
    g.record_scalar("acc", 0.7)
    g.flush([])
    assert abs(g.trend("acc").latest() - 0.6) < 1e-9


def test_collect_non_scalar_needs_reduce():
    g = FlowBuilder.from_(Scale(1.0)).tag("h").build()
    g.forward(V(torch.ones(2, 3)))
    with pytest.raises(Exception):
        g.collect(["h"])
    g.collect_with(["h"], Reduce.Mean)
    g.flush([])
    assert g.trend("h").latest() == 1.0


def test_flush_recurses_into_labeled_children():
    inner = FlowBuilder.from_(Scale(1.0)).through(MeanLoss()).tag("inner_loss").label("inner").build()
    outer = FlowBuilder.from_(inner).build()
    outer.forward(V(torch.ones(2)))
    outer.collect_at(["inner.inner_loss"])
    outer.flush([])
    assert outer.trend_at("inner.inner_loss").len() == 1


# ---- profiling / rendering ------------------------------------------------------------------------
def test_profiling_records_every_node():
    g = _mlp()
    g.enable_profiling()
    g.forward(V(torch.randn(2, 4)))
    prof = g.profile()
    assert prof is not None and len(prof.nodes) == 3 and prof.total > 0 and prof.timing("a") is not None
    g.collect_timings([])
    g.flush_timings([])
    g.disable_profiling()


def test_dot_contains_nodes_edges_and_tags():
    g = _mlp()
    dot = g.dot()
    assert dot.startswith("digraph") and "linear_1" in dot and "->" in dot and "#a" in dot


def test_end_step_and_epoch_counters():
    g = _mlp()
    g.end_step()
    g.end_step()
    g.end_epoch()
    assert g.step_count() == 2 and g.epoch_count() == 1


def test_graph_as_module_inside_graph_shares_parameters():
    inner = _mlp()
    outer = FlowBuilder.from_(inner).through(nn.Linear(2, 2)).build()
    assert len(outer.parameters()) == 6
    assert isinstance(outer.sub_modules()[0], Graph)


def test_native_topological_levels_match_python_rule():
    from flodl_b200 import _ext
    from flodl_b200.graph import topological_levels
    import pytest as _pytest
    assert topological_levels(5, [(0, 1), (0, 2), (1, 3), (2, 3), (0, 1), (3, 4)]) == [[0], [1, 2], [3], [4]]
    assert topological_levels(4, [(2, 0), (3, 0), (0, 1)]) == [[2, 3], [0], [1]]
    assert topological_levels(0, []) == []
    with _pytest.raises(Exception, match="cycle"):
        topological_levels(2, [(0, 1), (1, 0)])
    C = _ext.load()
    assert C is None or hasattr(C, "topo_levels")


# ---- the native (C++) walk and the Python walk are the same function --------------------------------------------------
def _both_walks(build, inputs, calls=2):
    """Outputs, tagged values and state after `calls` forwards, once through the C++ executor and once through the Python loop."""
    import os
    out = {}
    for native in ("1", "0"):
        os.environ["FLODL_B200_NATIVE_GRAPH"] = native
        try:
            torch.manual_seed(7)
            g = build()
            ys = [g.forward_multi(inputs).t.clone() for _ in range(calls)]
            assert (g._native_exec() is not None) == (native == "1")
            out[native] = (ys, {k: v.t.clone() for k, v in g.tagged_outputs.items()}, [s["value"].t.clone() for s in g.state if s["value"] is not None])
        finally:
            os.environ.pop("FLODL_B200_NATIVE_GRAPH", None)
    return out["1"], out["0"]


def test_native_walk_matches_python_walk_on_tags_state_refs_and_composites():
    from flodl_b200.graph import MergeOp, SoftmaxRouter, StateAdd

    def build():
        return (FlowBuilder.from_(nn.Linear(4, 8)).tag("stem").input(["extra"])
                .through(StateAdd()).using("memory")                     # forward reference: last call's value
                .split([nn.Linear(8, 8), nn.Linear(8, 8)]).tag_group("b").merge(MergeOp.Mean)
                .through(StateAdd()).using("extra")                      # a graph input used as a ref
                .gate(SoftmaxRouter(8, 2), [nn.Linear(8, 8), nn.Linear(8, 8)])
                .loop_body(FlowBuilder.new().also(nn.Linear(8, 8)).build()).for_n(2)
                .through(nn.Tanh()).tag("memory").through(nn.Linear(8, 2)).tag("out").build())
    x, extra = Variable.wrap(torch.randn(3, 4)), Variable.wrap(torch.randn(3, 8))
    (ya, ta, sa), (yb, tb, sb) = _both_walks(build, [x, extra], calls=3)
    assert all(torch.equal(a, b) for a, b in zip(ya, yb)) and not torch.equal(ya[0], ya[1])       # state moved between calls, identically
    assert ta.keys() == tb.keys() and set(ta) >= {"stem", "b_0", "b_1", "memory", "out"} and all(torch.equal(ta[k], tb[k]) for k in ta)
    assert len(sa) == len(sb) == 1 and torch.equal(sa[0], sb[0])


def test_native_walk_keeps_gradients_and_error_types():
    from flodl_b200.tensor import TensorError
    g = FlowBuilder.from_(nn.Linear(4, 4)).also(nn.Linear(4, 4)).through(nn.Linear(4, 1)).build()
    assert g._native_exec() is not None and g._native_exec().node_count() == len(g.nodes) and g._native_exec().level_count() == len(g.levels)
    x = Variable(torch.randn(5, 4), requires_grad=True)
    g.forward(x).sum().backward()
    assert x.grad() is not None and all(p.t.grad is not None for p in g.parameters())
    with pytest.raises(TensorError, match="expected 1 inputs, got 2"):
        g.forward_multi([x, x])

    class Boom(nn.Module):
        def forward(self, v): raise ValueError("inside a node")
    bad = FlowBuilder.from_(nn.Linear(4, 4)).through(Boom()).build()
    with pytest.raises(ValueError, match="inside a node"):                # a node's own exception passes through unchanged
        bad.forward(x)
    g.enable_profiling()                                                   # profiling uses the Python walk and still works
    g.forward(x)
    assert g.profile() is not None and len(g.profile().nodes) == len(g.nodes)
