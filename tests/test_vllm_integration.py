"""Plugin registration, runner path decisions and runner ops, with stand-in modules (no model load,
no dependence on the installed vLLM version)."""

import json
import sys
import types
from dataclasses import replace
from types import SimpleNamespace

import pytest
import torch

from conftest import SMALL
from moeflow_b200 import MoEConfig
from moeflow_b200.integrations import vllm_plugin, vllm_runner
from moeflow_b200.integrations.vllm_diagnostics import FixedLayerProbe, compare_outputs, compare_reduction_orders
from moeflow_b200.integrations.vllm_runner_ops import (
    combine_bf16_ring,
    compare_routing,
    fixed_capacity,
    local_to_global_ids,
    make_combine_fn,
    prepare_expert_inputs,
)
from moeflow_b200.utils.env import RunnerSettings


def _module(name, **attrs):
    mod = types.ModuleType(name)
    mod.__dict__.update(attrs)
    return mod


@pytest.fixture
def fake_vllm(monkeypatch):
    """A minimal ``vllm`` package tree in sys.modules with a factory-style MoE layer module."""
    def factory(*args, **kwargs):
        return ("layer", kwargs.get("runner_cls"))

    def original_pf(moe, quant_config, **kw):
        return "native_pf"

    tree = {
        "vllm": _module("vllm"),
        "vllm.model_executor": _module("vllm.model_executor"),
        "vllm.model_executor.layers": _module("vllm.model_executor.layers"),
        "vllm.model_executor.layers.fused_moe": _module("vllm.model_executor.layers.fused_moe", FusedMoEFactory=factory),
        "vllm.model_executor.layers.fused_moe.layer": _module("vllm.model_executor.layers.fused_moe.layer", FusedMoEFactory=factory),
        "vllm.model_executor.layers.fused_moe.all2all_utils": _module("vllm.model_executor.layers.fused_moe.all2all_utils", maybe_make_prepare_finalize=original_pf),
        "vllm.model_executor.layers.fused_moe.oracle": _module("vllm.model_executor.layers.fused_moe.oracle"),
        "vllm.model_executor.layers.fused_moe.oracle.fp8": _module("vllm.model_executor.layers.fused_moe.oracle.fp8", maybe_make_prepare_finalize=original_pf),
        "vllm.models": _module("vllm.models"),
        "vllm.models.glm5next": _module("vllm.models.glm5next"),
        "vllm.models.glm5next.common": _module("vllm.models.glm5next.common"),
        "vllm.models.glm5next.common.model": _module("vllm.models.glm5next.common.model", FusedMoEFactory=factory),
    }
    for name, mod in tree.items():
        monkeypatch.setitem(sys.modules, name, mod)
    sentinel_runner = type("SentinelRunner", (), {})
    monkeypatch.setattr(vllm_plugin, "_runner_class", lambda: sentinel_runner)
    return SimpleNamespace(tree=tree, factory=factory, original_pf=original_pf, runner=sentinel_runner)


def test_register_does_nothing_without_switches(monkeypatch, fake_vllm):
    monkeypatch.delenv("MOEFLOW_RUNNER", raising=False)
    monkeypatch.delenv("MOEFLOW_ALL2ALL", raising=False)
    vllm_plugin.register()
    assert fake_vllm.tree["vllm.model_executor.layers.fused_moe.layer"].FusedMoEFactory is fake_vllm.factory


def test_register_runner_wraps_every_binding_once(monkeypatch, fake_vllm):
    monkeypatch.setenv("MOEFLOW_RUNNER", "1")
    vllm_plugin.register()
    layer = fake_vllm.tree["vllm.model_executor.layers.fused_moe.layer"]
    pkg = fake_vllm.tree["vllm.model_executor.layers.fused_moe"]
    late = fake_vllm.tree["vllm.models.glm5next.common.model"]
    assert layer.FusedMoEFactory._moeflow_wrapped
    assert pkg.FusedMoEFactory is layer.FusedMoEFactory and late.FusedMoEFactory is layer.FusedMoEFactory
    wrapped = layer.FusedMoEFactory
    assert vllm_plugin.register_runner() == "already" and layer.FusedMoEFactory is wrapped
    assert layer.FusedMoEFactory(num_experts=4) == ("layer", fake_vllm.runner)
    chosen = object()
    assert layer.FusedMoEFactory(num_experts=4, runner_cls=chosen) == ("layer", chosen)


def test_register_runner_rebinds_runner_when_there_is_no_factory(fake_vllm):
    layer = fake_vllm.tree["vllm.model_executor.layers.fused_moe.layer"]
    del layer.FusedMoEFactory
    layer.MoERunner = type("MoERunner", (), {})
    assert vllm_plugin.register_runner() == "runner_binding"
    assert layer.MoERunner is fake_vllm.runner
    del layer.MoERunner
    with pytest.raises(RuntimeError):
        vllm_plugin.register_runner()


def test_prepare_finalize_is_patched_in_every_importable_call_site(monkeypatch, fake_vllm):
    patched = vllm_plugin.register_prepare_finalize()
    assert patched == ["all2all_utils", "fp8"]
    fn = fake_vllm.tree["vllm.model_executor.layers.fused_moe.oracle.fp8"].maybe_make_prepare_finalize
    assert fn._moeflow_wrapped_pf and vllm_plugin.register_prepare_finalize() == []
    no_a2a = SimpleNamespace(moe_parallel_config=SimpleNamespace(use_all2all_kernels=False, ep_size=1), num_local_experts=2)
    assert fn(no_a2a, None) == "native_pf"
    a2a = SimpleNamespace(moe_parallel_config=SimpleNamespace(use_all2all_kernels=True, ep_size=2), num_local_experts=2)
    assert fn(a2a, None, use_monolithic=True) == "native_pf"


def test_buffer_pool_is_keyed_by_configuration_and_dispatch_mode(monkeypatch):
    import moeflow_b200.fixed as fixed_mod

    monkeypatch.setattr(vllm_runner, "_BUFFER_POOL", {})
    monkeypatch.setattr(fixed_mod, "FixedEPLayer", lambda *a, **kw: SimpleNamespace(**kw))
    cfg, group = MoEConfig(), object()
    get = vllm_runner.shared_fixed_layer
    plain = get(cfg, 0, 4, 8, "cuda:0", group)
    assert get(cfg, 0, 4, 8, "cuda:0", group) is plain
    fused = get(cfg, 0, 4, 8, "cuda:0", group, fused_dispatch=True)
    assert fused is not plain and fused.fused_dispatch
    assert get(replace(cfg, top_k=4), 0, 4, 8, "cuda:0", group) is not plain
    assert get(cfg, 0, 4, 16, "cuda:0", group) is not plain


@pytest.mark.parametrize("local,counts,want", [(1, [1, 64], 64), (1, [1, 512], None), (0, [0, 0], 1), (5, None, 8), (256, [256], 256), (3, [2, 3], 4)])
def test_fixed_capacity_table(local, counts, want):
    assert fixed_capacity(local, counts, 256) == want


def test_settings_validation():
    assert RunnerSettings.from_env({}).mode == "route_check"
    s = RunnerSettings.from_env({"MOEFLOW_MODE": "fixed", "MOEFLOW_MAX_TOKENS": "64", "MOEFLOW_COMBINE_MODE": "bf16_ring",
                                 "MOEFLOW_FUSED_EXPERT_PREP": "1", "MOEFLOW_DIRECT_EXPERT_OUTPUT": "1"})
    assert (s.mode, s.max_tokens, s.combine_mode, s.direct_expert_output) == ("fixed", 64, "bf16_ring", True)
    for bad in ({"MOEFLOW_DIRECT_EXPERT_OUTPUT": "1"}, {"MOEFLOW_COMBINE_MODE": "fp16"}, {"MOEFLOW_MODE": "x"},
                {"MOEFLOW_VALIDATE_FIXED": "1"}, {"MOEFLOW_EXPERTS": "cublas"}):
        with pytest.raises(ValueError):
            RunnerSettings.from_env(bad)


class _FakeRunner(vllm_runner.RunnerCore):
    """RunnerCore on stand-ins for everything vLLM provides."""

    def __init__(self, settings, tokens_across_dp, monolithic=False, world=1):
        self.layer_name = "layers.0.mlp"
        self.native_calls, self.shared_calls = [], 0
        cfg = SMALL
        self.routed_experts = SimpleNamespace(
            quant_method=SimpleNamespace(is_monolithic=monolithic), w13_weight=None, w2_weight=None,
            global_num_experts=cfg.n_routed_experts, expert_map=None, activation="silu",
            forward_modular=lambda **kw: kw["x"] * 2,
        )
        self._quant_method = SimpleNamespace(topk_indices_dtype=torch.int32)
        self._shared_experts = None
        self.gate = SimpleNamespace(e_score_correction_bias=None)
        self.router = SimpleNamespace(select_experts=lambda **kw: __import__("moeflow_b200.router", fromlist=["route"]).route(kw["router_logits"], None, cfg))
        self._ctx = SimpleNamespace(dp_metadata=None if tokens_across_dp is None else SimpleNamespace(num_tokens_across_dp_cpu=torch.tensor(tokens_across_dp)), is_padding=None)
        self._group = SimpleNamespace(rank_in_group=0, world_size=world, device_group=None)
        self._moeflow_setup(cfg, settings)

    def _ep(self):
        return self._group

    def _forward_context(self):
        return self._ctx

    def _maybe_apply_shared_experts(self, *_):
        self.shared_calls += 1

    def _native_apply(self, hidden, *a, **kw):
        self.native_calls.append(hidden.shape[0])
        return None, hidden


def test_prefill_is_delegated_to_the_native_runner(tmp_path):
    r = _FakeRunner(RunnerSettings(mode="fixed", max_tokens=8, smoke_dir=tmp_path), [4, 64])
    x = torch.zeros(4, SMALL.hidden_size)
    r._apply_quant_method(x, torch.zeros(4, SMALL.n_routed_experts), None)
    assert r.native_calls == [4] and r._moeflow_fixed_calls == 0
    log = [json.loads(line) for line in (tmp_path / f"runner_pid{__import__('os').getpid()}.jsonl").read_text().splitlines()]
    assert log[0]["intercepted"] is False and log[0]["reason"] == "fixed token limit"


def test_monolithic_kernels_are_never_intercepted():
    r = _FakeRunner(RunnerSettings(mode="fixed"), [1, 1], monolithic=True)
    r._apply_quant_method(torch.zeros(1, SMALL.hidden_size), torch.zeros(1, SMALL.n_routed_experts), None)
    assert r.native_calls == [1]
    r = _FakeRunner(RunnerSettings(mode="route_check"), None, monolithic=True)
    r._apply_quant_method(torch.zeros(1, SMALL.hidden_size), torch.zeros(1, SMALL.n_routed_experts), None)
    assert r.native_calls == [1]


def test_route_check_uses_the_project_router_and_logs_agreement(tmp_path, monkeypatch):
    monkeypatch.setattr(vllm_runner, "_no_overlap_order", lambda: "NO_OVERLAP")
    r = _FakeRunner(RunnerSettings(mode="route_check", smoke_dir=tmp_path), None)
    x = torch.ones(3, SMALL.hidden_size)
    g = torch.Generator().manual_seed(0)
    shared, out = r._apply_quant_method(x, torch.randn(3, SMALL.n_routed_experts, generator=g), None)
    assert shared is None and torch.equal(out, x * 2) and r.shared_calls == 1
    log = [json.loads(line) for line in next(tmp_path.iterdir()).read_text().splitlines()]
    assert log[0]["token_expert_set_match"] == 1.0 and log[0]["max_abs_weight_diff_on_match"] == 0.0


def test_fixed_mode_runs_the_fixed_layer_on_cpu_with_external_experts(tmp_path, monkeypatch):
    """World 1 on CPU: the torch backend of the shared layer plus a stand-in for the engine's experts."""
    monkeypatch.setattr(vllm_runner, "_no_overlap_order", lambda: "NO_OVERLAP")
    monkeypatch.setattr(vllm_runner, "_BUFFER_POOL", {})
    r = _FakeRunner(RunnerSettings(mode="fixed", smoke_dir=tmp_path, fused_expert_prep=True), [3])
    seen = {}

    class Kernel:
        def apply(self, hidden_rows, w13, w2, weights, ids, **kw):
            seen["ids"], seen["weights"] = ids.clone(), weights.clone()
            return (hidden_rows.float() * weights.sum(-1, keepdim=True)).to(hidden_rows.dtype)

    r._local_kernel = Kernel()
    g = torch.Generator().manual_seed(1)
    x = torch.randn(3, SMALL.hidden_size, generator=g).bfloat16()
    logits = torch.randn(3, SMALL.n_routed_experts, generator=g)
    shared, out = r._apply_quant_method(x, logits, None)
    assert out.shape == x.shape and r._moeflow_fixed_calls == 1
    # world 1: every slot is local, so the weights of each row sum to the routed scaling factor
    torch.testing.assert_close(out.float(), (x.float() * SMALL.routed_scaling_factor).bfloat16().float(), rtol=2e-2, atol=2e-2)
    assert seen["ids"].shape == (4, SMALL.top_k)  # capacity 4 rows
    assert (seen["weights"][3] == 0).all()  # padding row: filler experts with zero weight
    log = [json.loads(line) for line in next(tmp_path.iterdir()).read_text().splitlines()]
    assert log[-1]["mode"] == "fixed" and log[-1]["capacity"] == 4 and log[-1]["experts"] == "vllm"


def test_routing_trace_is_gated_and_drops_padding(tmp_path):
    r = _FakeRunner(RunnerSettings(mode="route_check", routing_trace_dir=tmp_path), None)
    ids, w = torch.tensor([[1, 2], [3, 4], [5, 6]]), torch.rand(3, 2)
    r._record_routing_trace(ids, w)
    assert not list(tmp_path.glob("routes_*"))
    (tmp_path / "enabled").write_text("")
    r._ctx.is_padding = torch.tensor([False, True, False])
    r._record_routing_trace(ids, w)
    row = json.loads(next(tmp_path.glob("routes_*")).read_text())
    assert row["expert_ids"] == [[1, 2], [5, 6]] and row["execution_rows"] == 3 and row["padding_known"]
    r._ctx.is_padding = torch.tensor([False])
    with pytest.raises(ValueError):
        r._record_routing_trace(ids, w)


def test_local_to_global_ids_uses_a_foreign_filler():
    local = torch.tensor([[0, -1], [-1, 2]])
    w = torch.tensor([[0.5, 9.0], [float("nan"), 0.25]])
    gids, gw = local_to_global_ids(local, w, rank_offset=0, num_experts=16)
    assert gids.tolist() == [[0, 15], [15, 2]] and gw.tolist() == [[0.5, 0.0], [0.0, 0.25]]
    gids, _ = local_to_global_ids(local, w, rank_offset=8, num_experts=16)
    assert gids.tolist() == [[8, 0], [0, 10]]


def test_prepare_expert_inputs_ignores_garbage_in_invalid_rows():
    from moeflow_b200.fixed import FixedEPLayer
    from moeflow_b200.testing import make_weights

    cfg = SMALL
    w13, w2 = make_weights(cfg, 0)
    ly = FixedEPLayer(cfg, 0, 1, w13, w2, capacity=4, backend="torch")
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, cfg.hidden_size, generator=g).bfloat16()
    wts, ids = torch.rand(2, cfg.top_k, generator=g), torch.tensor([[1, 5], [7, 0]])
    ly.stage_dispatch_pack(x, wts, ids)
    ly._recv_store.copy_(ly._send_store)
    ly._recv_store[0, 3, : cfg.hidden_size] = float("nan")  # padding row payload
    rows = ly._recv_store.view(4, ly.pitch)[:, : ly.row_width]
    hidden, gids, weights = prepare_expert_inputs(rows, cfg.hidden_size, cfg.top_k, rank_offset=0, num_experts=cfg.n_routed_experts)
    assert gids[:2].tolist() == ids.tolist() and torch.equal(weights[:2], wts)
    assert gids[2:].tolist() == [[cfg.n_routed_experts - 1] * cfg.top_k] * 2 and (weights[2:] == 0).all()
    assert torch.equal(hidden[:2], x)


def test_ring_combine_witness_and_mode_factory():
    vals = torch.tensor([1.0, 256.0, 1.0, -256.0]).bfloat16().view(4, 1, 1)
    hit = torch.ones(1, 4, dtype=torch.bool)
    assert [combine_bf16_ring(vals, hit, r).item() for r in range(4)] == [1.0, 2.0, 2.0, 0.0]
    assert make_combine_fn("fp32", 0) is None and make_combine_fn("bf16_ring", 1).keywords == {"rank": 1}
    with pytest.raises(ValueError):
        make_combine_fn("fp64", 0)
    with pytest.raises(ValueError):
        combine_bf16_ring(vals.float(), hit, 0)
    # a masked owner contributes nothing, even when it holds NaN
    vals2 = vals.clone()
    vals2[2] = float("nan")
    hit2 = torch.tensor([[True, True, False, True]])
    assert combine_bf16_ring(vals2, hit2, 0).item() == 1.0


def test_compare_routing_ignores_slot_order():
    ids, w = torch.tensor([[3, 1], [0, 2]]), torch.tensor([[0.7, 0.3], [0.6, 0.4]])
    v_ids, v_w = torch.tensor([[1, 3], [0, 5]]), torch.tensor([[0.3, 0.7], [0.6, 0.4]])
    r = compare_routing(ids, w, v_ids, v_w)
    assert r["token_expert_set_match"] == 0.5 and r["max_abs_weight_diff_on_match"] == 0.0
    assert compare_routing(ids[:0], w[:0], v_ids[:0], v_w[:0]) == {"intercepted": True, "tokens": 0}


def test_diagnostics_compare_bytes_and_reduction_orders(tmp_path):
    pos, neg = torch.tensor([[0.0]]), torch.tensor([[-0.0]])
    r = compare_outputs(pos, neg)
    assert r["finite"] and r["max_abs_diff"] == 0 and not r["bitwise_equal"]
    assert not compare_outputs(torch.ones(1, 1), torch.ones(1, 1, dtype=torch.bfloat16))["bitwise_equal"]
    with pytest.raises(ValueError):
        compare_outputs(torch.ones(2, 1), torch.ones(2, 1), torch.tensor([True]))
    partials = torch.tensor([1.0, 256.0, 1.0, -256.0]).bfloat16().view(4, 1, 1)
    native = torch.tensor([[2.0]]).bfloat16()
    found = compare_reduction_orders(partials, native)
    assert found["tested"] == 1 + 24 + 3 and "bf16_order_2301" in found["exact_matches"]
    assert "fp32_then_bf16" in found["exact_matches"]  # 1 + 256 + 1 - 256 = 2 exactly in fp32
    assert compare_reduction_orders(torch.zeros(5, 1, 1), native)["tested"] == 0

    probe = FixedLayerProbe(tmp_path)
    experts = SimpleNamespace(forward_modular=lambda **kw: kw["x"] * 1.0)
    group = SimpleNamespace(rank_in_group=0, device_group=None)
    hidden = torch.ones(2, 4).bfloat16()
    args = (experts, hidden, torch.ones(2, 2), torch.tensor([[0, 1], [2, 3]]), hidden.clone(), "layers.0", 2)
    probe.compare(*args, ep_group=group)
    assert probe.calls == 0  # not enabled yet
    (tmp_path / "enabled").write_text("")
    for _ in range(3):
        probe.compare(*args, owner_partials=hidden.view(1, 2, 4), experts_per_rank=4, ep_group=group)
    rows = [json.loads(line) for line in next(tmp_path.glob("layer_comparison_*")).read_text().splitlines()]
    assert len(rows) == 2 and rows[0]["bitwise_equal"] and rows[0]["reduction_candidates"]["tested"] > 0


def test_router_without_an_id_dtype_argument_and_engine_without_forward_modular(monkeypatch):
    """The newer runner interface: ``select_experts`` takes no id dtype, the quant method applies the kernel."""
    monkeypatch.setattr(vllm_runner, "_no_overlap_order", lambda: "NO_OVERLAP")
    r = _FakeRunner(RunnerSettings(mode="route_check"), None)
    from moeflow_b200.router import route

    def select_experts(*, hidden_states, router_logits, input_ids=None):
        w, ids = route(router_logits, None, SMALL)
        return w, ids.to(torch.int64)

    r.router = SimpleNamespace(select_experts=select_experts)
    w, ids = r._select_experts(torch.zeros(2, SMALL.hidden_size), torch.randn(2, SMALL.n_routed_experts), None)
    assert ids.dtype == torch.int32 and r._router_takes_dtype is False
    applied = {}

    def apply(layer, x, topk_weights, topk_ids, shared_experts, shared_experts_input):
        applied["layer"] = layer
        return x * 3

    del r.routed_experts.forward_modular
    r._quant_method.apply = apply
    x = torch.ones(2, SMALL.hidden_size)
    shared, out = r._apply_quant_method(x, torch.randn(2, SMALL.n_routed_experts), None)
    assert torch.equal(out, x * 3) and applied["layer"] is r.routed_experts


def test_runner_class_follows_the_installed_engine_interface(monkeypatch):
    """Against the importable vLLM: the subclass takes ``layer`` first where the engine's runner does."""
    pytest.importorskip("vllm")
    import inspect

    try:
        from vllm.model_executor.layers.fused_moe.runner.moe_runner import MoERunner
    except ImportError:
        pytest.skip("this vLLM has no runner module")
    cls = vllm_runner.MoEFlowRunner
    assert issubclass(cls, MoERunner) and cls._moeflow_runner
    base_params = list(inspect.signature(MoERunner._apply_quant_method).parameters)
    ours = list(inspect.signature(cls._apply_quant_method).parameters)
    if "layer" not in base_params:
        assert ours[:4] == ["self", "hidden_states", "router_logits", "shared_experts_input"]
        return
    assert ours[: len(base_params)] == base_params
    # drive the layer-first entry with stand-ins: a prefill that the fixed mode declines goes to the engine's path
    runner = cls.__new__(cls)
    torch.nn.Module.__init__(runner)
    fake = _FakeRunner(RunnerSettings(mode="fixed", max_tokens=2), [4, 64])
    for name in ("layer_name", "_quant_method", "_shared_experts", "gate", "router"):
        runner.__dict__[name] = getattr(fake, name)
    runner._moeflow_setup(SMALL, RunnerSettings(mode="fixed", max_tokens=2))
    monkeypatch.setattr(cls, "_forward_context", lambda self: fake._ctx)
    seen = {}

    def engine_path(self, layer, hidden_states, router_logits, shared_experts_input, input_ids=None):
        seen["layer"] = layer
        return None, hidden_states + 1

    monkeypatch.setattr(MoERunner, "_apply_quant_method", engine_path)
    layer = fake.routed_experts
    x = torch.zeros(4, SMALL.hidden_size)
    shared, out = runner._apply_quant_method(layer=layer, hidden_states=x, router_logits=torch.zeros(4, SMALL.n_routed_experts),
                                             shared_experts_input=None)
    assert seen["layer"] is layer and runner.routed_experts is layer and torch.equal(out, x + 1)
    assert "routed_experts" not in dict(runner.named_children())


def test_row_transport_round_trip_and_reentry_guard():
    """World 1 with a loop-back exchange: every slot is local, ids come back global, the per-expert row counts
    are the histogram of the routing, and gather() merges the partial rows per token."""
    from moeflow_b200.integrations.row_transport import VariableRowTransport
    from moeflow_b200.router import route

    class Loopback:
        rank, world = 0, 1

        def exchange_counts(self, counts):
            return counts.clone()

        def exchange(self, rows, send_counts, recv_counts):
            return rows.clone()

    g = torch.Generator().manual_seed(4)
    x = torch.randn(5, SMALL.hidden_size, generator=g)
    w, ids = route(torch.randn(5, SMALL.n_routed_experts, generator=g), None, SMALL)
    t = VariableRowTransport(Loopback(), SMALL.n_routed_experts)
    got = t.scatter(x, w, ids, SMALL.n_routed_experts)
    assert t.busy and torch.equal(got.hidden, x) and torch.equal(got.expert_ids, ids) and torch.equal(got.weights, w)
    assert torch.equal(got.rows_per_local_expert.long(), torch.bincount(ids.flatten().long(), minlength=SMALL.n_routed_experts))
    with pytest.raises(RuntimeError, match="not re-entrant"):
        t.scatter(x, w, ids, SMALL.n_routed_experts)
    out = t.gather(got.hidden * got.weights.sum(dim=1, keepdim=True), torch.float32, wire_dtype=torch.float32)
    torch.testing.assert_close(out, x * w.sum(dim=1, keepdim=True))
    with pytest.raises(RuntimeError, match="without a matching"):
        t.gather(out, torch.float32)


def test_native_expert_kernels_are_chosen_by_weight_format():
    """bf16 weights and block-scaled e4m3 weights (fp32 scale per 128x128 block) run on this framework's own
    kernels; anything else keeps the engine's fused experts, or is an error when ``MOEFLOW_EXPERTS=native``."""
    r = _FakeRunner(RunnerSettings.from_env({"MOEFLOW_MODE": "fixed"}), [1])
    L, H, I = 2, 256, 128
    layer = SimpleNamespace(backend="cuda", L=L, H=H, I=I)
    bf16 = SimpleNamespace(w13_weight=torch.zeros(L, 2 * I, H, dtype=torch.bfloat16),
                           w2_weight=torch.zeros(L, H, I, dtype=torch.bfloat16))
    fp8 = SimpleNamespace(w13_weight=torch.zeros(L, 2 * I, H).to(torch.float8_e4m3fn),
                          w2_weight=torch.zeros(L, H, I).to(torch.float8_e4m3fn),
                          w13_weight_scale_inv=torch.ones(L, 2 * I // 128, H // 128),
                          w2_weight_scale_inv=torch.ones(L, H // 128, I // 128))
    per_tensor = SimpleNamespace(w13_weight=fp8.w13_weight, w2_weight=fp8.w2_weight,
                                 w13_weight_scale=torch.ones(L), w2_weight_scale=torch.ones(L))
    for experts, want in ((bf16, "bf16"), (fp8, "fp8"), (per_tensor, None)):
        r.routed_experts = experts
        assert r._use_native_experts(layer) == want
    r.routed_experts = fp8
    assert r._use_native_experts(SimpleNamespace(backend="torch", L=L, H=H, I=I)) is None
    r.moeflow = replace(r.moeflow, experts="native")
    r.routed_experts = per_tensor
    with pytest.raises(ValueError):
        r._use_native_experts(layer)
    r.moeflow = replace(r.moeflow, experts="vllm")
    r.routed_experts = bf16
    assert r._use_native_experts(layer) is None
