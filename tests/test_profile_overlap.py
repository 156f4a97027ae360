import json

from torchure_b200.train.profile_overlap import analyze, intersect_len, total_len, union


def test_interval_math():
    assert union([(0, 2), (1, 3), (5, 6)]) == [(0, 3), (5, 6)]
    assert total_len([(0, 3), (5, 6)]) == 4
    assert intersect_len([(0, 3), (5, 8)], [(2, 6)]) == 2


def test_analyze_classifies_our_comm_kernels(tmp_path):
    ev = lambda name, ts, dur, stream: {"ph": "X", "cat": "kernel", "name": name, "ts": ts, "dur": dur, "args": {"stream": stream}}
    trace = {"traceEvents": [
        ev("void tb::(anonymous namespace)::gemm_bf16_kernel<0,0,0>(...)", 0, 100, 7),
        ev("void tb::(anonymous namespace)::all_reduce_kernel<0>(...)", 50, 100, 9),   # 50 hidden, 50 exposed
        ev("ncclDevKernel_AllReduce_Sum_f32_RING_LL(...)", 200, 10, 11),                 # fully exposed
        ev("void tb::(anonymous namespace)::adamw_kernel(...)", 300, 50, 7),
    ]}
    p = tmp_path / "t.json"
    p.write_text(json.dumps(trace))
    res = analyze(str(p), steps=1)
    assert abs(res["compute_ms"] - 0.150) < 1e-9 and abs(res["comm_ms"] - 0.110) < 1e-9
    assert abs(res["hidden_ms"] - 0.050) < 1e-9 and abs(res["exposed_ms"] - 0.060) < 1e-9
    assert abs(res["idle_ms"] - 0.140) < 1e-9
