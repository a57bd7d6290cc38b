"""Statistics, decision rule, records, validation gates, serving validators, report generators."""

import json
import math

import pytest
import torch

from moeflow_b200.bench.logits import compare_logits, parse_raw_logits
from moeflow_b200.bench.record import make_record, write_record
from moeflow_b200.bench.stats import paired_ab, percentile, summarize, t95
from moeflow_b200.bench.validation import check_backend_pair, check_reference, require_matching_variants
from moeflow_b200.cli import summarize as S
from moeflow_b200.cli.smoke_client import compare, has_complete_logprobs, validate_prompts
from moeflow_b200.cli.validate_serving_result import METRICS, validate_result


def test_student_t_values():
    for df, want in ((1, 12.706), (2, 4.303), (9, 2.262), (19, 2.093), (30, 2.042)):
        assert abs(t95(df) - want) < 2e-3
    assert abs(t95(1000) - 1.962) < 2e-3
    with pytest.raises(ValueError):
        t95(0)


def test_percentile_and_summary():
    xs = [4.0, 1.0, 3.0, 2.0]
    assert percentile(xs, 0) == 1.0 and percentile(xs, 100) == 4.0 and percentile(xs, 50) == 2.5
    s = summarize(xs)
    assert s.n == 4 and s.median == 2.5 and s.min == 1.0 and abs(s.p95 - 3.85) < 1e-12
    assert summarize([7.0]).std == 0.0
    with pytest.raises(ValueError):
        percentile([], 50)


def test_paired_rule_needs_both_conditions():
    a = [100.0, 101.0, 99.5, 100.5, 100.2, 99.8]
    faster = [x - 5.0 for x in a]
    r = paired_ab(a, faster)
    assert r.significant and r.beneficial and r.mean_diff < 0 and r.ci95[1] < 0
    slower = paired_ab(faster, a)
    assert slower.significant and not slower.beneficial
    # a consistent but tiny gain does not beat the per-arm noise
    tiny = paired_ab(a, [x - 0.01 for x in a])
    assert not tiny.significant
    noisy_a = [100.0, 120.0, 80.0, 110.0, 90.0]
    noisy_b = [95.0, 118.0, 85.0, 100.0, 97.0]
    assert not paired_ab(noisy_a, noisy_b).significant
    with pytest.raises(ValueError):
        paired_ab([1.0], [1.0])


def test_records_are_self_describing_and_atomic(tmp_path):
    rec = make_record("unit", {"x": 1}, {"y": 2}, seed=3, complete=False)
    assert {"kind", "created", "complete", "git", "env", "seed", "command", "config", "results"} <= set(rec)
    assert "torch" in rec["env"] and "sha" in rec["git"]
    path = write_record(tmp_path / "deep" / "r.json", rec)
    assert json.loads(path.read_text())["complete"] is False and not list(path.parent.glob("*.tmp"))


def test_gates_reject_signed_zero_nan_and_errors():
    pos, neg = torch.tensor([[0.0]]), torch.tensor([[-0.0]])
    assert not check_backend_pair(pos, neg, pos)["bitwise_equal"]
    with pytest.raises(RuntimeError, match="outputs differ"):
        require_matching_variants(pos, neg)
    nan = torch.tensor([float("nan")])
    with pytest.raises(RuntimeError, match="outputs differ"):
        require_matching_variants(nan, nan.clone())
    require_matching_variants(torch.ones(3), torch.ones(3))
    ref = torch.randn(4, 8, generator=torch.Generator().manual_seed(0))
    good = check_reference(ref + 1e-4, ref)
    assert good["passed"] and good["tokens_checked"] == 4
    assert not check_reference(ref * 1.5, ref)["passed"]
    assert not check_reference(torch.full_like(ref, float("inf")), ref)["passed"]
    assert check_reference(ref[:0], ref[:0])["passed"]


def _serving_record(n=4, inp=8, outp=4, conc=2, duration=2.0):
    rec = {"num_prompts": n, "completed": n, "failed": 0, "max_concurrency": conc, "total_input_tokens": n * inp,
           "total_output_tokens": n * outp, "input_lens": [inp] * n, "output_lens": [outp] * n, "errors": [""] * n,
           "ttfts": [0.1] * n, "latencies": [0.5] * n, "itls": [[0.01] * (outp - 1)] * n, "duration": duration,
           "request_throughput": n / duration, "output_throughput": n * outp / duration}
    rec.update({m: 1.0 for m in METRICS})
    return rec


def test_serving_result_validator():
    ok = validate_result(_serving_record(), 4, 8, 4, 2)
    assert ok["passed"] and ok["total_output_tokens"] == 16 and ok["tokens_per_second"] == 8.0
    for mutate in (
        lambda r: r.update(completed=3),
        lambda r: r.update(output_lens=[4, 4, 4, 3]),
        lambda r: r.update(errors=["", "", "", "timeout"]),
        lambda r: r.update(median_tpot_ms=float("nan")),
        lambda r: r.pop("p99_itl_ms"),
        lambda r: r.update(itls=[[0.01]] * 3),
        lambda r: r.update(output_throughput=1.0),
        lambda r: r.update(ttfts=[0.1, 0.1, 0.1, -1.0]),
    ):
        rec = _serving_record()
        mutate(rec)
        with pytest.raises(ValueError):
            validate_result(rec, 4, 8, 4, 2)
    with pytest.raises(ValueError):
        validate_result(_serving_record(), 4, 8, 1, 2)


def test_smoke_client_validation_and_compare():
    assert validate_prompts(["a", [1, 2]]) == ["a", [1, 2]]
    for bad in ([], "x", [""], [[]], [[1, -2]], [[1.5]], [None]):
        with pytest.raises(ValueError):
            validate_prompts(bad)
    rec = {"prompt": "p", "dp_rank": 0, "text": "t", "tokens": ["a", "b"], "logprobs": [-0.1, -0.2], "complete": True}
    assert has_complete_logprobs(rec) and not has_complete_logprobs({**rec, "logprobs": [-0.1]})
    assert not has_complete_logprobs({**rec, "logprobs": [-0.1, math.inf]})
    a = {"records": [rec]}
    assert compare(a, {"records": [dict(rec)]})["passed"]
    assert not compare(a, {"records": [{**rec, "tokens": ["a", "c"]}]})["passed"]
    assert compare(a, {"records": [{**rec, "logprobs": [-0.1, -0.25]}]})["passed"]
    assert not compare(a, {"records": [{**rec, "logprobs": [-0.1, -0.25]}]}, exact_logprobs=True)["passed"]
    assert not compare(a, {"records": [{**rec, "complete": False}]})["passed"]
    assert not compare(a, {"records": []})["passed"]


def test_raw_logits_are_parsed_strictly():
    arr = parse_raw_logits([[0.5, 1.5, -2.0], [1.0, 2.0, 3.0]], 3)
    assert arr.shape == (2, 3) and arr.dtype.name == "float32"
    assert parse_raw_logits([0.5, 1.5, -2.0], 3).shape == (1, 3)
    with pytest.raises(ValueError):
        parse_raw_logits([[0.5, 1.5]], 3)
    with pytest.raises(ValueError):
        parse_raw_logits([[0.5, float("nan"), 1.0]], 3)
    same = compare_logits(arr, arr.copy())
    assert same["bitwise_equal"] and same["sha256_a"] == same["sha256_b"]
    other = arr.copy()
    other[0, 0] = -0.0 + 0.5000001
    assert not compare_logits(arr, other)["bitwise_equal"]
    assert not compare_logits(arr, arr[:1])["bitwise_equal"]


def test_report_generators_refuse_bad_records(tmp_path):
    pt = {"tokens": 8, "passed": True, "reference": [{"normwise_rel_err": 1e-3}],
          "graph_us": {"median": 10.0, "p95": 11.0}, "eager_us": {"median": 30.0}}
    rec = make_record("bench_layer", {"backend": "fused", "world": 2}, {"points": [pt]})
    good = write_record(tmp_path / "good.json", rec)
    assert "| fused | 2 | 8 | 10.0 | 11.0 | 30.0 |" in S.layer_table([str(good)])
    bad = write_record(tmp_path / "bad.json", {**rec, "complete": False})
    with pytest.raises(SystemExit):
        S.layer_table([str(bad)])
    failed = write_record(tmp_path / "failed.json", make_record("bench_layer", {"backend": "fused", "world": 2}, {"points": [{**pt, "passed": False}]}))
    with pytest.raises(SystemExit):
        S.layer_table([str(failed)])
    with pytest.raises(SystemExit):
        S.ab_table([str(good)])  # wrong kind
    csv_path = tmp_path / "launches.csv"
    csv_path.write_text('==PROF== header\n"ID","Kernel Name","Metric Name","Metric Unit","Metric Value"\n'
                        '"0","mf::combine_kernel(mf_combine_args)","gpu__time_duration.sum","ns","2,000"\n'
                        '"1","mf::combine_kernel(mf_combine_args)","gpu__time_duration.sum","ns","3,000"\n'
                        '"2","void at::native::fill(int)","gpu__time_duration.sum","ns","1,000"\n')
    text = S.launches_summary(str(csv_path))
    assert "mf::combine_kernel | 2 | 1.00 | 5.0" in text and "library helper kernels (at::native): 1" in text


def test_weight_source_specs_and_profiler_window():
    from moeflow_b200.bench.inputs import WeightSource, load_weights
    from moeflow_b200.bench.profiling import profile_layer
    from moeflow_b200.config import MoEConfig

    assert WeightSource.parse("synthetic") == WeightSource("synthetic")
    assert WeightSource.parse("real:17") == WeightSource("real", 17)
    for bad in ("", "real", "real:x", "synthetic:3", "file.pt"):
        with pytest.raises(ValueError):
            WeightSource.parse(bad)
    cfg = MoEConfig(hidden_size=16, moe_intermediate_size=8, n_routed_experts=4, top_k=2)
    w13, w2, bias = load_weights("synthetic", cfg, "cpu", experts=range(1, 3))
    assert w13.shape == (2, 16, 16) and w2.shape == (2, 16, 8) and bias.shape == (4,)
    with profile_layer("nothing to record", enabled=False) as window:
        assert not window.active


class _FakeCuda:
    """Enough of ``torch.cuda`` to run the timing helpers on a machine without a GPU: events read a counter
    that every "kernel" advances by one millisecond, graphs record the calls made during capture."""

    def __init__(self):
        self.clock_ms = 0.0
        self.log = []
        outer = self

        class Event:
            def __init__(self, enable_timing=False):
                self.at = None

            def record(self):
                self.at = outer.clock_ms

            def synchronize(self):
                pass

            def elapsed_time(self, other):
                return other.at - self.at

        class Stream:
            def wait_stream(self, other):
                pass

        class Graph:
            def __init__(self):
                self.calls = []

            def replay(self):
                for fn in self.calls:
                    fn()

        self.Event, self.Stream, self.CUDAGraph = Event, Stream, Graph
        self._capturing = None

    def synchronize(self):
        self.log.append("sync")

    def current_stream(self):
        return self.Stream()

    def stream(self, s):
        import contextlib

        return contextlib.nullcontext()

    def graph(self, g):
        import contextlib

        outer = self

        @contextlib.contextmanager
        def capturing():
            outer._capturing = g
            try:
                yield
            finally:
                outer._capturing = None

        return capturing()

    def kernel(self, tag):
        """A stand-in workload: runs now, or is recorded when a capture is open."""
        def body():
            self.clock_ms += 1.0
            self.log.append(tag)

        if self._capturing is not None:
            self._capturing.calls.append(body)
        else:
            body()


def test_timing_helpers_on_a_fake_device(monkeypatch):
    from moeflow_b200.bench import timing

    fake = _FakeCuda()
    for name in ("Event", "Stream", "CUDAGraph", "synchronize", "current_stream", "stream", "graph"):
        monkeypatch.setattr(torch.cuda, name, getattr(fake, name))
    flushes = []
    eager = timing.time_eager(lambda: fake.kernel("e"), reps=3, inner=4, warmup=2, flush=lambda: flushes.append(1))
    assert eager.mode == "eager" and eager.per_call_us == [1000.0] * 3 and len(flushes) == 3
    assert fake.log.count("e") == 2 + 3 * 4

    graphed = timing.time_graph(lambda: fake.kernel("g"), reps=2, inner=5, warmup=1)
    assert graphed.capturable and graphed.per_call_us == [1000.0, 1000.0]
    assert fake.log.count("g") == 1 + 5 * (1 + 2)  # warm-up call, one untimed replay, two timed replays

    def refuses():
        raise RuntimeError("operation not permitted when stream is capturing")

    failed = timing.time_graph(refuses, reps=2, inner=2, warmup=0)
    assert not failed.capturable and failed.per_call_us == [] and "not permitted" in failed.error

    a, b = timing.time_graphs_alternating(lambda: fake.kernel("A"), lambda: (fake.kernel("B"), fake.kernel("B")), reps=3, inner=1)
    assert a == [1000.0] * 3 and b == [2000.0] * 3
    order = [t for t in fake.log if t in "AB"]
    assert order[-9:] == ["A", "B", "B"] * 3  # strictly alternating


def test_headline_bench_clock_summary_and_cli_defaults():
    """``bench.py`` is importable without a GPU; its clock sampler turns nvidia-smi lines into the median SM
    clock, the maximum clock and the set of active throttle reasons."""
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("headline_bench", Path(__file__).resolve().parent.parent / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)

    sampler = bench.ClockSampler(0)
    assert sampler.stop()["reasons"] == ["nvidia-smi unavailable"]  # never started

    class Quiet:
        def terminate(self): pass
        def wait(self, timeout=None): return 0

    sampler.proc = Quiet()
    sampler.lines = [
        "1965, 1965, 310.5, Not Active, Not Active, Not Active, Not Active",
        "1350, 1965, 998.0, Not Active, Not Active, Not Active, Active",
        "1410, 1965, 870.2, Not Active, Not Active, Not Active, Not Active",
        "garbage line",
        "[N/A], 1965, 1.0, Not Active, Not Active, Not Active, Not Active",
    ]
    summary = sampler.stop()
    assert summary == {"sm_mhz": 1410.0, "sm_max_mhz": 1965.0, "power_w_max": 998.0, "samples": 3, "reasons": ["sw_power_cap"]}


def test_pair_and_decode_tables(tmp_path):
    gate = {"a": {"passed": True}, "b": {"passed": True}}
    paired = {"median_improvement": 28.7, "ci95": [-30.1, -27.0], "significant": True, "beneficial": True}
    pt = {"tokens": 1, "gate": gate, "a_us": {"median": 141.9}, "b_us": {"median": 113.2}, "paired": paired}
    rec = make_record("ab_native_fixed", {"a": "vllm_agrs", "b": "fused", "world": 2}, {"points": [pt]})
    good = write_record(tmp_path / "pair.json", rec)
    assert "| vllm_agrs | fused | 2 | 1 | 141.9 | 113.2 | +28.7 |" in S.ab_table([str(good)])
    failed = write_record(tmp_path / "pair_failed.json", make_record(
        "ab_native_fixed", {"a": "vllm_agrs", "b": "fused", "world": 2},
        {"points": [{**pt, "gate": {"a": {"passed": True}, "b": {"passed": False}}}]}))
    with pytest.raises(SystemExit):
        S.ab_table([str(failed)])

    dpt = {"concurrency": 4, "batch_per_rank": 1, "tpot_ms": {"median": 8.7456, "p95": 8.7579}, "tokens_per_second": 457.4,
           "status": {"code": 0, "name": "ok"}, "finite": True}
    drec = make_record("decode_bench", {"layers": 42, "world": 4, "fp8": True}, {"points": [dpt]})
    dgood = write_record(tmp_path / "decode.json", drec)
    assert "| 42 | 4 | e4m3 | 4 | 1 | 8.746 | 8.758 | 457 |" in S.decode_table([str(dgood)])
    dbad = write_record(tmp_path / "decode_bad.json", make_record(
        "decode_bench", {"layers": 42, "world": 4, "fp8": False},
        {"points": [{**dpt, "status": {"code": 3, "name": "dispatch flag wait ran out"}}]}))
    with pytest.raises(SystemExit):
        S.decode_table([str(dbad)])
    with pytest.raises(SystemExit):
        S.decode_table([str(good)])  # wrong kind
