"""Host logic of the serving harnesses (no engine, no GPU): the summary rows of the throughput run and the
latency statistics of the closed loop."""

import pytest

from echokv_b200.harness import latency, throughput


def test_throughput_summary_ratios_against_stock():
    rows = {"stock": {"kv_capacity_tokens": 1000, "output_tok_s": 50.0},
            "echokv-int4": {"kv_capacity_tokens": 3100, "output_tok_s": 60.0},
            "echokv-int8": {"error": "exit 1"}}
    rep = throughput.summarize(rows)
    assert rep["failed"] == ["echokv-int8"]
    assert rep["rows"]["echokv-int4"]["capacity_vs_stock"] == pytest.approx(3.1)
    assert rep["rows"]["echokv-int4"]["output_tok_s_vs_stock"] == pytest.approx(1.2)
    assert set(throughput.CONFIGS) >= {"stock", "echokv-int4", "echokv-int8", "echokv-live-mem4", "echokv-live-mem6"}


def test_latency_statistics_of_a_closed_loop():
    # two requests: first token after 0.5 s / 0.2 s, then one token every 0.1 s / 0.05 s
    reqs = [{"arrival": 10.0, "token_times": [10.5, 10.6, 10.7, 10.8]},
            {"arrival": 20.0, "token_times": [20.2, 20.25, 20.3]},
            {"arrival": 30.0, "token_times": []}]  # never produced a token: not counted
    s = latency.summarize_requests(reqs, wall=2.0)
    assert s["completed"] == 2 and s["output_tok_s"] == pytest.approx(3.5)
    assert s["ttft"]["mean_ms"] == pytest.approx(350.0) and s["ttft"]["p99_ms"] == pytest.approx(500.0)
    assert s["tpot"]["mean_ms"] == pytest.approx(75.0)
    assert s["itl"]["median_ms"] == pytest.approx(100.0) and len(latency.METRICS) == 4
    assert s["e2el"]["p99_ms"] == pytest.approx(800.0)
    assert latency.percentiles([])["mean_ms"] is None


def test_closed_loop_keeps_the_concurrency_and_serves_every_prompt():
    class Out:
        def __init__(self, rid, n, fin):
            self.request_id, self.finished = rid, fin
            self.outputs = [type("O", (), {"token_ids": list(range(n))})()]

    class Engine:  # one token per running request per step, three tokens per request
        def __init__(self):
            self.running, self.max_running, self.served = {}, 0, 0

        def add_request(self, rid, prompt, params):
            self.running[rid] = 0
            self.max_running = max(self.max_running, len(self.running))

        def step(self):
            outs = []
            for rid in list(self.running):
                self.running[rid] += 1
                done = self.running[rid] == 3
                outs.append(Out(rid, self.running[rid], done))
                if done:
                    del self.running[rid]
                    self.served += 1
            return outs

    eng = Engine()
    res = latency.closed_loop(eng, [{"prompt_token_ids": [1]}] * 7, None, concurrency=3)
    assert eng.served == 7 and eng.max_running == 3 and res["completed"] == 7
    assert res["output_tok_s"] * res["wall_s"] == pytest.approx(21)

    class DeltaEngine(Engine):  # reports only the tokens of the step
        def step(self):
            outs = super().step()
            for o in outs:
                o.outputs[0].token_ids = o.outputs[0].token_ids[-1:]
            return outs

    eng = DeltaEngine()
    res = latency.closed_loop(eng, [{"prompt_token_ids": [1]}] * 5, None, concurrency=2, delta=True)
    assert eng.served == 5 and res["output_tok_s"] * res["wall_s"] == pytest.approx(15)
