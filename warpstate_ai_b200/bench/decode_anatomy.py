"""What a decode step is made of, without a profiler.

``parts``   CUDA graphs of SUBSETS of one step's launches (the four projections, the attention step, the two
            residual+norm kernels) over all layers of the 2.005 B model at batch 64, each replayed back to back and
            timed with CUDA events.  The results of a subset are meaningless (its inputs are stale), its time is
            not: the parts add up to the whole step, so each kernel's share is what its own graph takes.
``tail``    The persistent layer-tail launch (`torch.ops.ws_b200.decode_layer_tail`) against the six launches it
            replaces, on six distinct layers of weights (larger than L2): time per layer eager and inside a CUDA
            graph, and the launch's own phase boundaries from the ``%globaltimer`` stamps every CTA writes into the
            optional ``trace`` tensor.

    python -m warpstate_ai_b200.bench.decode_anatomy parts [--batch 64] [--position 64] [--only attention]
    python -m warpstate_ai_b200.bench.decode_anatomy tail  [--batch 64]

One JSON line per measurement.
"""
from __future__ import annotations

import argparse
import json

import torch


def timed_graph(fn, replays: int = 50) -> float:
    """Milliseconds per replay of a CUDA graph of ``fn`` (captured after two warm-up calls on a side stream)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
        fn()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    for _ in range(5):
        graph.replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(replays):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / replays


def timed_eager(fn, repeats: int = 10) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / repeats


def parts(batch: int, position: int = 0, only=None) -> None:
    from .. import WarpStateLM, warpstate_2b
    from ..serve.engine import DecodeEngine
    torch.manual_seed(0)
    with torch.device("cuda"):
        model = WarpStateLM(warpstate_2b())
    model.eval().requires_grad_(False)
    engine = DecodeEngine(model, dtype=torch.bfloat16)
    engine.new_state(batch)
    engine.pos_dev.fill_(position)      # the attention step reads the cache rows below this in-chunk position
    k, ops = engine._kbufs, torch.ops.ws_b200
    d, ffn, eps, pos = engine.cfg.d_model, engine.cfg.ffn_hidden, engine.cfg.rms_eps, engine.pos_dev

    def step(chosen) -> None:
        for w, st in zip(engine.weights, engine.states):
            if "in_proj" in chosen:
                ops.decode_gemm(w["w_in"], k["n"], 5 * d, 0, k["qkvgu"], k["flag"], False)
            if "attention" in chosen:
                ops.decode_attn(k["qkvgu"], st.k, st.v, st.u, st.mixed, k["rope"], pos, engine.h, k["y"])
            if "out_proj" in chosen:
                ops.decode_gemm(w["w_out"], k["y"], d, 1, k["p_out"], k["flag"], False)
            if "norm" in chosen:
                ops.decode_reduce_norm(k["x"], k["p_out"], None, None, None, None, w["n2"], eps, k["n"])
            if "up_gate" in chosen:
                ops.decode_gemm(w["w_ug"], k["n"], ffn, 2, k["act"], k["flag"], False)
            if "down" in chosen:
                ops.decode_gemm(w["w_down"], k["act"], d, 1, k["p_down"], k["flag"], False)
            if "norm" in chosen:
                ops.decode_reduce_norm(k["x"], k["p_down"], None, None, None, None, w["n2"], eps, k["n"])

    everything = ["in_proj", "attention", "out_proj", "norm", "up_gate", "down"]
    subsets = (everything, ["in_proj", "out_proj", "up_gate", "down"], ["attention", "norm"], ["in_proj"], ["up_gate"],
               ["out_proj"], ["down"], ["attention"], ["norm"])
    for chosen in subsets if only is None else [only.split(",")]:
        print(json.dumps({"launches": chosen, "layers": len(engine.weights), "batch": batch, "in_chunk_position": position,
                          "ms_per_step": round(timed_graph(lambda: step(chosen)), 4)}), flush=True)


def tail(batch: int) -> None:
    from ..ops import _ext
    _ext.require()
    ops = torch.ops.ws_b200
    torch.manual_seed(0)
    dev = torch.device("cuda")
    d, ffn, layers = 2048, 7168, 6
    weights = [{name: (torch.randn(rows, cols, device=dev) * 0.02).bfloat16()
                for name, (rows, cols) in (("out", (d, d)), ("ug", (2 * ffn, d)), ("down", (d, ffn)), ("inp", (5 * d, d)))}
               for _ in range(layers)]
    x = torch.randn(batch, d, device=dev)
    y = torch.randn(batch, d, device=dev).bfloat16()
    n = torch.zeros(batch, d, device=dev, dtype=torch.bfloat16)
    act = torch.zeros(batch, ffn, device=dev, dtype=torch.bfloat16)
    qkvgu = torch.zeros(batch, 5 * d, device=dev, dtype=torch.bfloat16)
    p_out = torch.zeros(ops.decode_gemm_splits(d, d), batch, d, device=dev)
    p_down = torch.zeros(ops.decode_gemm_splits(d, ffn), batch, d, device=dev)
    norm_w, scale, bias = torch.ones(d, device=dev), torch.zeros(d, device=dev), torch.zeros(d, device=dev)
    barrier = torch.zeros(2, dtype=torch.int32, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    traces = [torch.zeros(sms, 16, dtype=torch.long, device=dev) for _ in range(layers)]

    def persistent(trace: bool = False) -> None:
        for i, w in enumerate(weights):
            ops.decode_layer_tail(w["out"], w["ug"], w["down"], weights[(i + 1) % layers]["inp"], y, x, p_out, p_down, n, act,
                                  qkvgu, norm_w, scale, bias, norm_w, 1e-5, barrier, flag, traces[i] if trace else None)

    def six_launches() -> None:
        for i, w in enumerate(weights):
            ops.decode_gemm(w["out"], y, d, 1, p_out, flag, False)
            ops.decode_reduce_norm(x, p_out, None, None, None, None, norm_w, 1e-5, n)
            ops.decode_gemm(w["ug"], n, ffn, 2, act, flag, False)
            ops.decode_gemm(w["down"], act, d, 1, p_down, flag, False)
            ops.decode_reduce_norm(x, p_down, None, None, scale, bias, norm_w, 1e-5, n)
            ops.decode_gemm(weights[(i + 1) % layers]["inp"], n, 5 * d, 0, qkvgu, flag, False)

    for name, fn in (("persistent launch", persistent), ("six launches", six_launches)):
        print(json.dumps({"arm": name, "us_per_layer_eager": round(timed_eager(fn) * 1e3 / layers, 2),
                          "us_per_layer_in_graph": round(timed_graph(fn, 10) * 1e3 / layers, 2), "batch": batch,
                          "error_flag": int(flag[0])}), flush=True)
    persistent(trace=True)
    torch.cuda.synchronize()
    names = ["start", "out_proj stored", "barrier 1", "norm 1", "barrier 2", "up/gate stored", "barrier 3", "down stored",
             "barrier 4", "norm 2", "barrier 5", "in_proj stored"]
    stamps = traces[layers // 2].cpu()[:, :12].double()
    relative = (stamps - stamps[:, 0].min()) / 1e3
    print(json.dumps({"phase_boundaries_us": {names[j]: {"min": round(float(relative[:, j].min()), 2),
                                                         "median": round(float(relative[:, j].median()), 2),
                                                         "max": round(float(relative[:, j].max()), 2)} for j in range(12)}}),
          flush=True)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["parts", "tail"])
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--position", type=int, default=0, help="parts: in-chunk position of the step (0..127)")
    ap.add_argument("--only", default=None, help="parts: one comma-separated subset instead of the standard ones")
    a = ap.parse_args()
    if a.what == "parts":
        parts(a.batch, a.position, a.only)
    else:
        tail(a.batch)


if __name__ == "__main__":
    main()
