"""Per-kernel timings of the layer's stages against their rooflines.

    python -m omni_moe_b200.kernel_bench [--config c2|c3|c4|c5|all] [--reps N] [--backward]

For each stage of a configuration the script launches the kernel through the C ABI inside a CUDA
graph (several launches per replay, so host launch cost does not count), times replays with CUDA
events and prints one JSON line: microseconds per launch, the algorithmic work of the launch and
the fraction of the measured peak (HBM copy bandwidth or bf16 tensor throughput from
MEASURED_PEAKS.json at the repository root; a stated fallback if the file is absent).

Configurations (synthetic data, seeded):
  c2  quick-start layer: T 4096, H 1024, I 4096, 64x64 experts, k 16
  c3  router microbench: T 16384, H 2048, 256x256 experts, k 16
  c4  skewed expert stress: T 32768, H 2048, 512x512 experts, k 32, Zipf(1.1) routing
  c5  large table: T 65536, H 4096, I 11008, 1024x1024 experts, k 64 (needs ~25 GB of device memory)
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np
import torch

from . import _lib
from .ops.scheduler import workspace_bytes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CONFIGS = {
    "c2": dict(T=4096, H=1024, I=4096, n=64, k=16, zipf=None),
    "c3": dict(T=16384, H=2048, I=0, n=256, k=16, zipf=None),
    "c4": dict(T=32768, H=2048, I=0, n=512, k=32, zipf=1.1),
    "c5": dict(T=65536, H=4096, I=11008, n=1024, k=64, zipf=None),
}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def _randn_bf16(shape, std, dev, seed):
    """Large bf16 normal tensors, generated on the device in slabs to bound temporary memory."""
    g = torch.Generator(device=dev).manual_seed(seed)
    out = torch.empty(shape, device=dev, dtype=torch.bfloat16)
    rows = shape[0]
    step = max(1, (64 << 20) // max(1, shape[1]))
    for s in range(0, rows, step):
        e = min(rows, s + step)
        out[s:e] = (torch.randn((e - s, shape[1]), device=dev, generator=g) * std).to(torch.bfloat16)
    return out


def _zipf_indices(t, k, n_experts, s, seed, dev):
    rng = np.random.default_rng(seed)
    p = np.arange(1, n_experts + 1, dtype=np.float64) ** (-s)
    cdf = np.cumsum(p / p.sum())
    u = rng.random((t, k))
    return torch.from_numpy(np.minimum(np.searchsorted(cdf, u), n_experts - 1).astype(np.int32)).to(dev)


def time_graph(fn, launches=4, reps=10):
    """Microseconds per launch of `fn(stream_ptr)`, measured over graph replays."""
    fn(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for _ in range(launches):
                fn(s.cuda_stream)
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3 / launches)
    ts.sort()
    return ts[len(ts) // 2]


def time_graph_cold(fn, reps=10):
    """Microseconds of one launch of `fn(stream_ptr)` that finds nothing of its data in L2: a 512 MB fill runs before
    every launch, and the fill's own time (measured the same way) is taken off."""
    dev = torch.device("cuda", torch.cuda.current_device())
    junk = torch.empty(512 << 20, device=dev, dtype=torch.uint8)

    def flush_then(run_fn):
        def go(stream_ptr):
            junk.fill_(1)
            if run_fn:
                fn(stream_ptr)
        return go
    both = time_graph(flush_then(True), launches=1, reps=reps)
    alone = time_graph(flush_then(False), launches=1, reps=reps)
    return both - alone


def run_backward(name: str, reps: int):
    """Stages of the backward pass (router scatter, expert gradients, MLP gradient GEMMs and helpers)."""
    from .ops.scheduler import schedule
    c = CONFIGS[name]
    T, H, I, n, k = c["T"], c["H"], c["I"], c["n"], c["k"]
    N, P = n * n, T * k
    dev = torch.device("cuda", torch.cuda.current_device())
    hbm, tf, src = peaks()
    lib = _lib.load()
    chk = _lib.check
    i32 = dict(device=dev, dtype=torch.int32)
    f32 = dict(device=dev, dtype=torch.float32)
    bf = dict(device=dev, dtype=torch.bfloat16)
    status = torch.zeros(1, **i32)

    def report(stage, us, bound, work, note=""):
        ach = work / (us * 1e-6) / (1e9 if bound == "hbm" else 1e12)
        line = dict(config=name, stage=stage, us=round(us, 2), bound=bound)
        if bound == "hbm":
            line.update(algorithmic_bytes=int(work), achieved_gbs=round(ach, 1), peak_gbs=hbm, frac=round(ach / hbm, 3))
        else:
            line.update(flops=int(work), achieved_tflops=round(ach, 1), peak_tflops=tf, frac=round(ach / tf, 3))
        line["peak_source"] = src
        if note:
            line["note"] = note
        print(json.dumps(line), flush=True)

    x = _randn_bf16((T, H), 1.0, dev, 0)
    dy = _randn_bf16((T, H), 0.1, dev, 9)
    if c["zipf"]:
        indices = _zipf_indices(T, k, N, c["zipf"], 0, dev)
    else:
        indices = torch.randint(0, N, (T, k), device=dev, dtype=torch.int32, generator=torch.Generator(device=dev).manual_seed(3))
    weights = torch.rand((T, k), **f32)
    U = int(torch.unique(indices).numel())
    # ---- router scatter -------------------------------------------------------------------------
    dsc = torch.randn((T, k), **f32)
    dlx, dly = torch.empty((T, n), **f32), torch.empty((T, n), **f32)
    us = time_graph(lambda s: chk(lib.omni_router_bwd(dsc.data_ptr(), indices.data_ptr(), 0, T, n, k, dlx.data_ptr(),
                                                      dly.data_ptr(), status.data_ptr(), s)), reps=reps)
    report("router_bwd_scatter", us, "hbm", 8.0 * P + 8.0 * T * n)
    # ---- routed experts ---------------------------------------------------------------------------
    up = _randn_bf16((N, H), 0.02, dev, 3)
    down = _randn_bf16((N, H), 0.02, dev, 4)
    ds, cd, dg = torch.empty((T, k), **f32), torch.empty((T, k), **f32), torch.empty((T, k), **f32)
    us = time_graph(lambda s: chk(lib.omni_expert_bwd_dots(x.data_ptr(), up.data_ptr(), down.data_ptr(), dy.data_ptr(),
                                                           weights.data_ptr(), indices.data_ptr(), T, k, H, N, ds.data_ptr(),
                                                           cd.data_ptr(), dg.data_ptr(), None, _lib.OMNI_BF16, status.data_ptr(), s)), reps=reps)
    report("expert_bwd_dots", us, "hbm", 4.0 * T * H + 4.0 * U * H + 20.0 * P, f"U={U} distinct experts; gathers 2 rows per pair")
    dx = torch.empty((T, H), **bf)
    us = time_graph(lambda s: chk(lib.omni_expert_combine(up.data_ptr(), ds.data_ptr(), indices.data_ptr(), T, k, H, N, None,
                                                          dx.data_ptr(), _lib.OMNI_BF16, status.data_ptr(), s)), reps=reps)
    report("expert_bwd_dx (combine kernel)", us, "hbm", 2.0 * T * H + 2.0 * U * H + 8.0 * P)
    sch = schedule(indices, N, segments=True)
    cap = sch.expert_ids.numel()
    d_up, d_dn = torch.empty((cap, H), **bf), torch.empty((cap, H), **bf)
    scratch = torch.empty(int(lib.omni_expert_bwd_rows_scratch_bytes(P, H)), device=dev, dtype=torch.uint8)
    for label, sc in (("expert_bwd_rows", scratch), ("expert_bwd_rows (one warp per segment)", None)):
        if sc is None and c["zipf"]:
            continue  # a 100k-pair segment on one warp takes a large fraction of a second
        us = time_graph(lambda s: chk(lib.omni_expert_bwd_rows(
            x.data_ptr(), dy.data_ptr(), ds.data_ptr(), cd.data_ptr(), sch.sorted_pair_ids.data_ptr(), sch.expert_ids.data_ptr(),
            sch.offsets.data_ptr(), sch.meta.data_ptr(), sch.meta[1:].data_ptr(), cap, T, k, H, 1, d_up.data_ptr(), d_dn.data_ptr(), _lib.OMNI_BF16,
            _lib.ptr(sc), sc.numel() if sc is not None else 0, status.data_ptr(), s)), reps=reps)
        report(label, us, "hbm", 4.0 * T * H + 4.0 * U * H + 12.0 * P, "compact rows; gathers 2 token rows per pair")
    # ---- shared MLP ---------------------------------------------------------------------------------
    if I:
        Tp = (T + 7) // 8 * 8
        gu = _randn_bf16((T, 2 * I), 1.0, dev, 5)
        dact = _randn_bf16((T, I), 0.1, dev, 6)
        dgu, dgu_t, act_t = torch.empty((T, 2 * I), **bf), torch.empty((2 * I, Tp), **bf), torch.empty((I, Tp), **bf)
        us = time_graph(lambda s: chk(lib.omni_swiglu_bwd(gu.data_ptr(), dact.data_ptr(), T, I, dgu.data_ptr(), dgu_t.data_ptr(),
                                                          act_t.data_ptr(), Tp, s)), reps=reps)
        report("swiglu_bwd (+ transposed outputs)", us, "hbm", 2.0 * (3 * T * I + 2 * T * I + 3 * T * I))
        wt = torch.empty((I, H), **bf)
        wd = _randn_bf16((H, I), I ** -0.5, dev, 7)
        us = time_graph(lambda s: chk(lib.omni_transpose_bf16(wd.data_ptr(), H, I, I, wt.data_ptr(), H, H, s)), reps=reps)
        report("transpose [H, I]", us, "hbm", 4.0 * H * I)
        x_t = torch.empty((H, Tp), **bf)
        dy_t = torch.empty((H, Tp), **bf)
        wgu_t = _randn_bf16((H, 2 * I), H ** -0.5, dev, 8)
        out_ti, out_th = torch.empty((T, I), **bf), torch.empty((T, H), **bf)
        out_hi, out_2ih = torch.empty((H, I), **bf), torch.empty((2 * I, H), **bf)
        gemms = (("gemm dact = dy Wd", dy, wt, out_ti), ("gemm dx = dgu (Wg;Wu)", dgu, wgu_t, out_th),
                 ("gemm dWd = dy^T act", dy_t, act_t, out_hi), ("gemm dWgu = dgu^T x", dgu_t, x_t, out_2ih))
        for label, a, b, o in gemms:
            m_, k_ = a.shape
            n_ = b.shape[0]
            us = time_graph(lambda s: chk(lib.omni_gemm_bf16_nt(a.data_ptr(), b.data_ptr(), m_, n_, k_, o.data_ptr(), n_,
                                                                status.data_ptr(), s)), reps=reps)
            report(label, us, "tensor", 2.0 * m_ * n_ * k_, f"{m_} x {n_} x {k_}")
        # the same four products with the operands read in place (transposed ones as MN-major tiles): what the
        # MLP backward runs by default
        act = torch.empty((T, I), **bf)
        us = time_graph(lambda s: chk(lib.omni_swiglu_bwd_limit(gu.data_ptr(), dact.data_ptr(), T, I, 0.0, dgu.data_ptr(), None, None,
                                                                0, act.data_ptr(), s)), reps=reps)
        report("swiglu_bwd (dgate | dup and act, no transposed copies)", us, "hbm", 2.0 * (3 * T * I + 2 * T * I + T * I))
        wgu = _randn_bf16((2 * I, H), H ** -0.5, dev, 9)
        xb = _randn_bf16((T, H), 1.0, dev, 10)
        in_place = (("gemm dact = dy Wd, Wd in place", dy, 0, wd, 1, T, I, H, out_ti),
                    ("gemm dx = dgu (Wg;Wu), weights in place", dgu, 0, wgu, 1, T, H, 2 * I, out_th),
                    ("gemm dWd = dy^T act, both in place", dy, 1, act, 1, H, I, T, out_hi),
                    ("gemm dWgu = dgu^T x, both in place", dgu, 1, xb, 1, 2 * I, H, T, out_2ih))
        for label, a, at, b, bt, m_, n_, k_, o in in_place:
            us = time_graph(lambda s: chk(lib.omni_gemm_bf16(a.data_ptr(), at, a.stride(0), b.data_ptr(), bt, b.stride(0), m_, n_, k_,
                                                             o.data_ptr(), n_, status.data_ptr(), s)), reps=reps)
            report(label, us, "tensor", 2.0 * m_ * n_ * k_, f"{m_} x {n_} x {k_}")
    torch.cuda.synchronize()
    if int(status.item()):
        raise RuntimeError("a kernel reported a device-side fault: " + _lib.status_message(int(status.item())))


def run_config(name: str, reps: int):
    c = CONFIGS[name]
    T, H, I, n, k = c["T"], c["H"], c["I"], c["n"], c["k"]
    N, P = n * n, T * k
    dev = torch.device("cuda", torch.cuda.current_device())
    hbm, tf, src = peaks()
    lib = _lib.load()
    chk = _lib.check
    i32 = dict(device=dev, dtype=torch.int32)
    f32 = dict(device=dev, dtype=torch.float32)
    status = torch.zeros(1, **i32)
    x = _randn_bf16((T, H), 1.0, dev, 0)
    kx = _randn_bf16((n, H), H ** -0.5, dev, 1)
    ky = _randn_bf16((n, H), H ** -0.5, dev, 2)
    logits = torch.empty((T, 2 * n), **f32)
    scores, weights = torch.empty((T, k), **f32), torch.empty((T, k), **f32)
    indices = torch.empty((T, k), **i32)
    out = []

    def report(stage, us, bound, work, note=""):
        if bound == "hbm":
            ach = work / (us * 1e-6) / 1e9
            line = dict(config=name, stage=stage, us=round(us, 2), bound="hbm", algorithmic_bytes=int(work),
                        achieved_gbs=round(ach, 1), peak_gbs=hbm, frac=round(ach / hbm, 3))
        else:
            ach = work / (us * 1e-6) / 1e12
            line = dict(config=name, stage=stage, us=round(us, 2), bound="tensor", flops=int(work),
                        achieved_tflops=round(ach, 1), peak_tflops=tf, frac=round(ach / tf, 3))
        line["peak_source"] = src
        if note:
            line["note"] = note
        print(json.dumps(line), flush=True)
        out.append(line)

    # ---- router gates (tensor) -----------------------------------------------------------------
    us = time_graph(lambda s: chk(lib.omni_router_gate(x.data_ptr(), kx.data_ptr(), ky.data_ptr(), T, H, n,
                                                       logits.data_ptr(), status.data_ptr(), s)), reps=reps)
    report("router_gate_gemm", us, "tensor", 4.0 * T * H * n)
    # ---- BatchNorm / log-softmax / top-k (hbm) -------------------------------------------------
    us = time_graph(lambda s: chk(lib.omni_router_logits_topk(logits.data_ptr(), 2 * n, None, None, T, n, k,
                                                              scores.data_ptr(), indices.data_ptr(), 0,
                                                              weights.data_ptr(), None, s)), reps=reps)
    report("router_logits_topk", us, "hbm", 2.0 * T * n * 4 + T * k * 12)
    # ---- routing for the expert stages ----------------------------------------------------------
    if c["zipf"]:
        indices.copy_(_zipf_indices(T, k, N, c["zipf"], 0, dev))
        weights.copy_(torch.distributions.Dirichlet(torch.ones(k)).sample((T,)).to(dev))
    U = int(torch.unique(indices).numel())
    # ---- scheduling (hbm) ---------------------------------------------------------------------
    ws = torch.empty(workspace_bytes(P, N), device=dev, dtype=torch.uint8)
    perm, sorted_e = torch.empty(P, **i32), torch.empty(P, **i32)
    meta = torch.zeros(4, **i32)
    us = time_graph(lambda s: chk(lib.omni_schedule(indices.data_ptr(), 0, None, 0, T, k, N, perm.data_ptr(),
                                                    sorted_e.data_ptr(), None, None, None, None, meta.data_ptr(),
                                                    ws.data_ptr(), ws.numel(), s)), reps=reps)
    report("schedule_permutation", us, "hbm", 20.0 * P + 8.0 * N, "bytes per the full description (20 P + 8 N)")
    # same-box bar: the library sort the reference's scheduler calls (torch.sort, stable, on the flat expert ids)
    flat_ids = indices.view(-1)
    us_t = time_graph(lambda s: torch.sort(flat_ids, stable=True), launches=1, reps=reps) if P else 0.0
    report("schedule_bar_torch_stable_sort", us_t, "hbm", 20.0 * P + 8.0 * N, "torch.sort(stable=True) of the same keys, for comparison")
    # ---- routed experts (hbm): algorithmic bytes = x in, y out, each touched Up/Down row once, schedule arrays
    up = _randn_bf16((N, H), 0.02, dev, 3)
    down = _randn_bf16((N, H), 0.02, dev, 4)
    coef = torch.empty((T, k), **f32)
    y = torch.empty((T, H), device=dev, dtype=torch.bfloat16)
    alg = 4.0 * T * H + 4.0 * U * H + 12.0 * P
    us_c = time_graph(lambda s: chk(lib.omni_expert_coef(x.data_ptr(), up.data_ptr(), weights.data_ptr(), perm.data_ptr(),
                                                         sorted_e.data_ptr(), T, k, H, N, coef.data_ptr(),
                                                         status.data_ptr(), s)), reps=reps)
    us_b = time_graph(lambda s: chk(lib.omni_expert_combine(down.data_ptr(), coef.data_ptr(), indices.data_ptr(), T, k, H, N,
                                                            None, y.data_ptr(), _lib.OMNI_BF16, status.data_ptr(), s)),
                      reps=reps)
    report("expert_coef", us_c, "hbm", 2.0 * T * H + 2.0 * U * H + 12.0 * P, f"U={U} distinct experts")
    # the same with the hot experts' products from one dense GEMM (what the scheduled path launches from 4096 tokens)
    hot_ws = torch.empty(int(lib.omni_expert_coef_hot_workspace(T, H)), device=dev, dtype=torch.uint8)
    us_h = time_graph(lambda s: chk(lib.omni_expert_coef_hot(x.data_ptr(), up.data_ptr(), weights.data_ptr(), perm.data_ptr(),
                                                             sorted_e.data_ptr(), T, k, H, N, 0, coef.data_ptr(),
                                                             hot_ws.data_ptr(), hot_ws.numel(), status.data_ptr(), s)),
                      reps=reps)
    n_hot = int(hot_ws[256:260].view(torch.int32).item())
    report("expert_coef_hot", us_h, "hbm", 2.0 * T * H + 2.0 * U * H + 12.0 * P, f"{n_hot} experts treated densely")
    report("expert_combine", us_b, "hbm", 2.0 * T * H + 2.0 * U * H + 8.0 * P)
    report("expert_coef+combine", us_c + us_b, "hbm", alg, f"gather traffic through L2: {2.0 * P * H * 2 / 2**30:.2f} GiB")
    if H <= 2048:
        us = time_graph(lambda s: chk(lib.omni_expert_fused(x.data_ptr(), up.data_ptr(), down.data_ptr(), weights.data_ptr(),
                                                            indices.data_ptr(), T, k, H, N, None, y.data_ptr(),
                                                            _lib.OMNI_BF16, None, status.data_ptr(), s)), reps=reps)
        report("expert_fused", us, "hbm", alg - 12.0 * P + 8.0 * P)
    from .ops.expert import use_routed_kernel
    if H <= 2048 and n <= 256 and use_routed_kernel(N, H, n, k):
        # selection + routed experts in one kernel, from the router logits (what the layer launches for tables in L2)
        logits_r = torch.randn((T, 2 * n), **f32)
        sc_r, w_r = torch.empty((T, k), **f32), torch.empty((T, k), **f32)
        idx_r = torch.empty((T, k), **i32)
        run_routed = lambda s: chk(lib.omni_route_expert_fused(
            logits_r.data_ptr(), 2 * n, None, None, x.data_ptr(), up.data_ptr(), down.data_ptr(), T, n, k, H, N, y.data_ptr(),
            y.data_ptr(), sc_r.data_ptr(), idx_r.data_ptr(), w_r.data_ptr(), status.data_ptr(), s))
        us = time_graph(run_routed, reps=reps)
        u_r = int(torch.unique(idx_r).numel())
        alg_r = 6.0 * T * H + 4.0 * u_r * H + 8.0 * T * n + 12.0 * P   # x in, y in and out, touched rows once, logits in, routing out
        report("route_expert_fused_warm", us, "hbm", alg_r, f"tables in L2; {u_r} distinct experts")
        report("route_expert_fused_cold", time_graph_cold(run_routed, reps=reps), "hbm", alg_r, "L2 flushed before every launch")
    # ---- shared MLP (tensor) --------------------------------------------------------------------
    if I:
        wg = _randn_bf16((I, H), H ** -0.5, dev, 5)
        wu = _randn_bf16((I, H), H ** -0.5, dev, 6)
        wd = _randn_bf16((H, I), I ** -0.5, dev, 7)
        act = torch.empty((T, I), device=dev, dtype=torch.bfloat16)
        us = time_graph(lambda s: chk(lib.omni_mlp_gate_up(x.data_ptr(), wg.data_ptr(), wu.data_ptr(), T, H, I,
                                                           act.data_ptr(), status.data_ptr(), s)), reps=reps)
        report("mlp_gate_up_swiglu", us, "tensor", 4.0 * T * H * I)
        us = time_graph(lambda s: chk(lib.omni_mlp_down(act.data_ptr(), wd.data_ptr(), T, H, I, None, y.data_ptr(),
                                                        status.data_ptr(), s)), reps=reps)
        report("mlp_down", us, "tensor", 2.0 * T * H * I)
    torch.cuda.synchronize()
    if int(status.item()) or int(meta[2].item()):
        raise RuntimeError("a kernel reported a device-side fault: " + _lib.status_message(int(status.item()) | int(meta[2].item())))
    return out


def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", default="c2", choices=[*CONFIGS, "all"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--backward", action="store_true", help="time the backward kernels instead of the forward ones")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("kernel_bench needs a CUDA device")
    for name in (CONFIGS if args.config == "all" else [args.config]):
        (run_backward if args.backward else run_config)(name, args.reps)
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
