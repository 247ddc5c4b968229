"""Host-side fault hooks, the device-status watchdog, profiler back ends and the request trace log."""
import json

import pytest
import torch

from xllm_b200 import LLM, SamplingParams
from xllm_b200.engine.fault import DeviceWatchdog, FaultPlan
from xllm_b200.utils.tracing import Profiler, TraceLog, nvtx_range


def test_fault_plan_parsing_and_rank_selection():
    p = FaultPlan.parse("worker_exit@step=3@rank=1, slow_rank_ms=5, rpc_drop=1.0", rank=1)
    assert p.exit_step == 3 and p.slow_ms == 5 and p.drop()
    other = FaultPlan.parse("worker_exit@step=3@rank=1", rank=0)
    assert other.exit_step is None
    slept = []
    p.before_step(0, sleep=slept.append)
    assert slept == [0.005]
    with pytest.raises(SystemExit):
        p.before_step(3, sleep=slept.append)
    with pytest.raises(ValueError):
        FaultPlan.parse("gpu_hang")                       # only host-side faults exist


def test_engine_raises_at_the_planned_step(monkeypatch):
    monkeypatch.setenv("XLLM_FAULT", "raise@step=2")
    llm = LLM("tiny", devices="cpu", dtype="float32", num_blocks=64, enable_graph=False)
    llm.engine.add_request("a", list(range(5, 25)), max_tokens=8, temperature=0.0, ignore_eos=True)
    llm.engine.step()
    llm.engine.step()
    with pytest.raises(RuntimeError, match="XLLM_FAULT"):
        llm.engine.step()
    llm.engine.fault = None                               # the engine itself is intact: the request completes
    toks = []
    while llm.engine.has_unfinished():
        toks += [e.token for e in llm.engine.step() if e.token >= 0]
    assert len(toks) >= 5


def test_watchdog_marks_unhealthy_with_the_reason():
    state = {"gemm": 0, "comm": 0}
    seen = []
    wd = DeviceWatchdog({"gemm": lambda: state["gemm"], "tp_comm": lambda: state["comm"]}, seen.append)
    assert wd.check() and not seen
    state["comm"] = 7                                     # what a kernel leaves behind when a bounded wait expired
    assert not wd.check()
    assert "tp_comm" in seen[0] and "status 7" in seen[0]

    def broken():
        raise OSError("device lost")
    wd2 = DeviceWatchdog({"attention": broken}, seen.append)
    assert not wd2.check() and "unreadable" in seen[-1]


def test_profiler_backends_and_trace_log(tmp_path):
    with nvtx_range("noop on cpu"):
        pass
    p = Profiler("torch", rank=3)
    p.start()
    torch.ones(8).sum()
    path = p.stop(str(tmp_path))
    assert path.endswith(".pt.trace.json") and "xllm_rank3_" in path and json.load(open(path))["traceEvents"] is not None
    c = Profiler("cuda")
    c.start()
    assert c.stop() == ""
    with pytest.raises(ValueError):
        Profiler("perf")
    off = TraceLog("")
    off.event("r", "arrive")                              # disabled: nothing happens
    log = TraceLog(str(tmp_path / "trace.log"))
    log.event("r1", "arrive", prompt_tokens=5)
    log.event("r1", "finish", reason="length")
    log.close()
    lines = [json.loads(x) for x in open(tmp_path / "trace.log")]
    assert [x["event"] for x in lines] == ["arrive", "finish"] and lines[0]["prompt_tokens"] == 5


def test_sampling_is_reproducible_for_a_seed():
    """Same seed twice -> the same tokens, also with temperature, top-p and top-k in play."""
    outs = []
    for _ in range(2):
        llm = LLM("tiny", devices="cpu", dtype="float32", num_blocks=64, enable_graph=False, seed=11)
        sp = SamplingParams(max_tokens=12, temperature=0.9, top_p=0.9, top_k=50, ignore_eos=True, seed=123)
        outs.append([o.outputs[0].token_ids for o in llm.generate([list(range(3, 20)), list(range(40, 49))], sp)])
    assert outs[0] == outs[1]
