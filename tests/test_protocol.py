"""Host logic of the measuring / checking protocol (decide_b200/protocol.py) on the CPU: the quantile rule of the
reference's bench (crates/decide-cli/src/bench.rs:103-112; its own test 518-530 compares with numpy), the machine-state
capture against faked command output, the FLAG rules (bench.rs:466-474), the parity table (check.rs:270-343)."""
import numpy as np

from decide_b200 import protocol as P


def test_quantile_is_numpys_linear_interpolation():
    rs = np.random.RandomState(0)
    for n in (1, 2, 5, 10, 20):
        x = rs.rand(n) * 100
        for q in (0.0, 0.5, 0.95, 1.0):
            assert abs(P.quantile(x, q) - np.percentile(x, 100 * q)) < 1e-9
    assert np.isnan(P.quantile([], 0.5))
    s = P.stats([3.0, 1.0, 2.0])
    assert (s["p50"], s["min"], s["max"], s["mean"], s["samples"]) == (2.0, 1.0, 3.0, 2.0, [3.0, 1.0, 2.0])   # every sample is kept


def _fake(outputs):
    def run(cmd):
        for key, out in outputs.items():
            if key in " ".join(cmd):
                return out
        return None
    return run


def test_machine_state_and_flags():
    quiet = _fake({"ps -Ao": " 12.5 /usr/bin/python3\n  0.5 bash\n",
                   "--query-gpu": "NVIDIA B200, 1965, 1965, 180.20, 1000.00, 1024, 183359, Not Active, Not Active, Not Active, Not Active\n",
                   "--query-compute-apps": ""})
    m = P.machine_state(0, run=quiet)
    assert m["gpu"]["name"] == "NVIDIA B200" and m["gpu"]["sm_max_mhz"] == 1965.0 and m["gpu"]["throttle_reasons"] == []
    assert m["gpu"]["other_processes"] == 0 and not m["gpu_flag"]
    assert m["top_processes"][0] == {"cpu_percent": 12.5, "process": "python3"}
    assert isinstance(m["cores"], int) and "B200" in P.describe_machine(m)
    calm = dict(m, load_flag=False)
    assert P.flags(calm, calm) == []
    hot = P.machine_state(0, run=_fake({"--query-gpu": "NVIDIA B200, 1100, 1965, 990.0, 1000.00, 1, 2, Not Active, Active, Not Active, Active\n",
                                        "--query-compute-apps": "4242, 1000\n"}))
    assert hot["gpu"]["throttle_reasons"] == ["hw_thermal_slowdown", "sw_power_cap"] and hot["gpu"]["other_processes"] == 1 and hot["gpu_flag"]
    fl = P.flags(dict(calm, load_flag=True), hot, encoded_during_runs=3, allocations_during_runs=1)
    assert any("load above 1 per core" in f for f in fl)
    assert any("hw_thermal_slowdown" in f and "after" in f for f in fl) and not any("sw_power_cap" in f for f in fl)   # the power cap is normal
    assert any("other compute process" in f for f in fl)
    assert any("3 tensor maps were encoded during the runs" in f for f in fl) and any("1 device allocations" in f for f in fl)
    nothing = P.machine_state(0, run=lambda cmd: None)      # no nvidia-smi, no ps: still a record
    assert nothing["gpu"]["name"] is None and nothing["top_processes"] == []


def test_check_table_rules():
    rs = np.random.RandomState(1)
    want = rs.randn(6, 16).astype(np.float32) * 3
    ncand = np.full(6, 16, np.uint32)
    good = dict(name="ticket-like", tokens=603, rows=597, got=want + 0.004, want=want, ncand=ncand, forward_ms=9.2)
    ok, lines = P.check_table([good])
    assert ok and any("summary: 1 requests, 6 fields: PASS" in l for l in lines)
    off = want.copy()
    off[2, 3] += 0.5                                       # a logit far outside the bar
    ok, lines = P.check_table([good, dict(good, name="bad", got=off)])
    assert not ok and any(l.strip().startswith("bad:") for l in lines) and any("FAIL" in l for l in lines)
    tie = want.copy()                                      # a near-tie: top two 0.01 apart, the engine flips them
    tie[0, :2] = [5.0, 4.99]
    tie[0, 2:] = -5.0
    flipped = tie.copy()
    flipped[0, :2] = [4.992, 4.998]
    ok, lines = P.check_table([dict(good, name="tie", got=flipped, want=tie)])
    assert ok and any("flips below the 0.05 gold margin (allowed): tie:" in l for l in lines)


def test_measure_request_cold_and_follow_up():
    """bench.rs:209-290: a cold measurement empties the state cache before every run; a follow-up runs its primer once
    and never forgets."""
    from types import SimpleNamespace

    from decide_b200 import protocol

    calls = []

    class FakeEngine:
        def forget_states(self):
            calls.append("forget")

    class FakeDecisionEngine:
        engine = FakeEngine()

        def decide(self, text):
            calls.append(text)
            return SimpleNamespace(prepared=SimpleNamespace(ids=[0] * 40), rows=17, route="snapshot" if text == "primer" else "state_cache",
                                   response={"answers": {"team": {"decision": "billing"}}}, timings={"tokenize_ms": 0.1, "forward_ms": 2.0, "head_ms": 0.05})

    cold = protocol.measure_request(FakeDecisionEngine(), "card", "req", iters=4, warmup=3)
    assert calls == ["forget", "req"] * 7 and cold["kind"] == "cold" and cold["forward_ms"]["p50"] == 2.0 and len(cold["e2e_ms"]["samples"]) == 4
    assert cold["decisions"] == {"team": "billing"} and cold["tokens"] == 40 and cold["rows"] == 17
    calls.clear()
    warm = protocol.measure_request(FakeDecisionEngine(), "card", "req", iters=4, warmup=3, primer="primer")
    assert calls == ["primer"] + ["req"] * 7 and warm["kind"] == "follow-up" and warm["route"] == "state_cache"
