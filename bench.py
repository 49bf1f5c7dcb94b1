#!/usr/bin/env python
"""Benchmark of the leaf-parallel evaluation path on B200.

One "step" = one leaf batch through the hot path: Gomoku 15x15 positions ->
bf16 input planes (encoder kernel) -> 10 x 64 residual tower + policy / value
heads.  Headline metric: network leaf evaluations per second.

  value     all ranks' evaluations / max-over-ranks device time, inputs (move
            histories) already resident in HBM, outputs left in HBM.
  e2e       the same through the host-buffer call a user makes
            (ob200_net_infer_gomoku): host -> device copies of the histories
            and device -> host copies of policy + value inside the timed region.
  roofline  the dominant kernel (3x3 convolution, tensor-core bound): algorithmic
            FLOPs of one launch / its average duration, against the measured
            bf16 peak; timed live on a ping-pong loop of the very kernel.
  selection batched PUCT selection + virtual-loss apply + revert over 65,536
            nodes x 225 children (HBM bound), timed in the same run.
  cpu_baseline  the reference's own CPU code (oracle/_ref: libtorch forward +
            GomokuState encoder; else the oracle port) on a bounded sample.

`--impl reference` times that CPU path alone with the same JSON keys.
Multi-GPU: one process per GPU (torchrun), independent replicas, no data-path
collective; per-GPU counters are summed after the timed region.
"""
import argparse
import contextlib
import io
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from omoknuni_small_b200 import replicas, synth  # noqa: E402

NET = dict(board_size=15, input_channels=17, filters=64, blocks=10, policy_size=225, policy_head_ch=2,
           value_head_ch=1, value_hidden=256)
SEL_NODES, SEL_CHILDREN = 65536, 225
SELW_NODES, SELW_CHILDREN = 2048, 4672      # chess-wide child rows (154 MB per pass)
METRIC, UNIT = "nn_leaf_evals_per_sec", "evals/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_burst=p["bf16_tflops"], bf16_sustained=p.get("bf16_tflops_sustained"),
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16_burst=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop = index, [], threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        while not self.stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                self.rows.append([c.strip() for c in out.strip().split(",")])
            except Exception:
                pass
            self.stop.wait(0.2)

    def __enter__(self):
        self.thread.start()
        return self

    def __exit__(self, *a):
        self.stop.set()
        self.thread.join(timeout=6)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_baseline(steps, warmup, sample_b=256):
    """The reference's CPU path on a bounded sample: encode + forward of `sample_b` positions per step."""
    from oracle import capi as oc, net_ref
    shapes = synth.net_tensor_shapes(NET["board_size"], NET["input_channels"], NET["filters"], NET["blocks"],
                                     NET["policy_size"], NET["policy_head_ch"], NET["value_head_ch"])
    w = synth.make_weights(shapes, seed=42, init="kaiming_normal")
    games, hist, nh, tm = synth.make_gomoku_games(sample_b, 15, seed=1000)
    cores = os.cpu_count() or 1
    kind = "reference" if (oc.have_ref_net() and oc.have_ref_tree()) else "port"
    times = []
    if kind == "reference":
        # The reference class hard-codes 32-channel heads; the benchmark network has 2 / 1, so the
        # reference class runs the tower it shares with the benchmark network and its own heads.
        net = oc.RefNet(17, 15, NET["blocks"], 64, 225, seed=42)
        for k, a in w.items():
            if k.startswith(("input_", "res_blocks")):
                net.set(k, a)
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            planes, _ = oc.ref_gomoku_encode_batch(games, 15, threads=cores)
            net.forward(np.ascontiguousarray(planes[:, :17]), threads=cores)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
        what = (f"{sample_b} positions/step: reference GomokuState::getEnhancedTensorRepresentation (OpenMP) + "
                f"ResNetModel::forward (libtorch CPU fp32, 32/32 heads), {cores} threads")
    else:
        for i in range(warmup + steps):
            t0 = time.perf_counter()
            planes = oc.gomoku_encode(hist, nh, tm, 15, 17, threads=cores)
            net_ref.forward(w, planes, threads=cores)
            if i >= warmup:
                times.append(time.perf_counter() - t0)
        what = f"{sample_b} positions/step: oracle port (C encoder + torch CPU fp32 forward), {cores} threads"
    sec = float(np.mean(times))
    return {"value": sample_b / sec, "unit": UNIT, "cores": cores, "kind": kind, "sample": what}, sec


def selection_cpu_baseline(n_nodes=4096):
    """MCTSNode::selectChild + applyVirtualLoss + revertVirtualLoss on real reference nodes (or the port)."""
    from oracle import capi as oc
    t = synth.make_selection_tree(n_nodes, SEL_CHILDREN, seed=7)
    cores = os.cpu_count() or 1
    if oc.have_ref_tree():
        _, _, _, secs = oc.ref_select(t, repeats=5, threads=cores)
        return {"value": n_nodes * 5 / secs, "unit": "selections/s", "cores": cores, "kind": "reference",
                "sample": f"{n_nodes} parents x 225 children, 5 passes, real MCTSNode objects, OpenMP over parents"}
    t0 = time.perf_counter()
    for _ in range(5):
        s = oc.puct_select(t, apply_vl=True, threads=cores)
        oc.vl_revert(t, s, 3)
    return {"value": n_nodes * 5 / (time.perf_counter() - t0), "unit": "selections/s", "cores": cores, "kind": "port",
            "sample": f"{n_nodes} parents x 225 children, 5 passes, flat-array port"}


def arm_config(B, world):
    """The workload both arms report."""
    return {"workload": "gomoku15x15 leaf batch: encode + resnet 10x64 (2/1-channel heads) forward",
            "leaf_batch_per_gpu": B, "l2": "flushed between timed steps (256 MB write)",
            "replicas": world, "weights": "kaiming-normal seed 42, BN identity"}


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base, sec = cpu_baseline(args.steps, max(1, min(args.warmup, 2)))
    line = {"metric": METRIC, "value": base["value"], "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(arm_config(args.batch, args.gpus), sample_batch=256,
                           note="the reference class hard-codes 32/32-channel heads; one step = a 256-position sample of the leaf batch"),
            "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


WIDE_NETS = [
    dict(name="go19x19 resnet 20x128, policy FC 362 (2/1-channel heads)", S=19, cin=17, F=128, blocks=20, A=362, pc=2, vc=1,
         kind=0, B=2048, scalar=0),
    dict(name="chess8x8 resnet 20x256, 119 planes, 73 policy planes (4672 logits)", S=8, cin=119, F=256, blocks=20, A=4672,
         pc=73, vc=1, kind=1, B=4096, scalar=7),
]


def time_wide_net(capi, torch, wc, dev, local, rank, flush, timed, steps):
    """Forward of one wide-tower configuration on a device-resident input board tensor, and its
    dominant kernel (F -> F convolution with residual) alone."""
    S, F, B = wc["S"], wc["F"], wc["B"]
    shapes = synth.net_tensor_shapes(S, wc["cin"], F, wc["blocks"], wc["A"], wc["pc"], wc["vc"], policy_planes=wc["kind"] == 1)
    w = synth.make_weights(shapes, seed=42, init="torch_default", bn="random")
    net = capi.Net(wc["cin"], S, wc["blocks"], F, wc["A"], wc["pc"], wc["vc"], 256, B, local, policy_kind=wc["kind"]).load(w)
    rng = np.random.default_rng(replicas.shard_seed(3000, rank))
    planes = (rng.random((B, wc["cin"], S, S)) < 0.1).astype(np.float32)
    if wc["scalar"]:
        planes[:, wc["cin"] - wc["scalar"]:] = rng.random((B, wc["scalar"], S, S)).astype(np.float32)
    bt = capi.planes_to_board_tensor(torch.from_numpy(planes).to(dev), net.input_tensor_channels())
    pol = torch.empty((B, wc["A"]), dtype=torch.float32, device=dev)
    val = torch.empty(B, dtype=torch.float32, device=dev)

    def fwd():
        net.forward_device(bt, B, pol, val, capi.OUT_PROBS)
    for _ in range(3):
        fwd()
    ms = float(np.mean(timed(fwd, steps)))
    rngw = np.random.default_rng(0)
    wp = torch.from_numpy(capi.pack_conv3x3(rngw.normal(0, 0.03, (F, F, 3, 3)).astype(np.float32), None, F).view(np.int16)).to(dev)
    bias = torch.zeros(F, device=dev)
    n_el = int(capi.lib().ob200_board_tensor_bytes(S, B, F)) // 2
    bufs = [torch.zeros(n_el, dtype=torch.int16, device=dev) for _ in range(3)]
    reps = 10

    def conv_loop():
        for i in range(reps):
            capi.conv3x3(bufs[i % 3], wp, bias, bufs[(i + 2) % 3], B, S, F, F, True, out=bufs[(i + 1) % 3])
    conv_loop()
    conv_ms = float(np.mean(timed(conv_loop, 3))) / reps
    net.close()
    return dict(cfg=wc, ms=ms, conv_ms=conv_ms)


def wide_report(wr, world, peaks):
    wc = wr["cfg"]
    S2 = wc["S"] * wc["S"]
    if wc["kind"] == 1:     # convolutional policy head: 1x1 convolution to the planes, no FC
        flops = (synth.net_flops_per_eval(wc["S"], wc["cin"], wc["F"], wc["blocks"], 0, 0, wc["vc"])
                 + 2 * S2 * wc["F"] * wc["pc"])
    else:
        flops = synth.net_flops_per_eval(wc["S"], wc["cin"], wc["F"], wc["blocks"], wc["A"], wc["pc"], wc["vc"])
    conv_tf = 2.0 * S2 * 9 * wc["F"] * wc["F"] * wc["B"] / (wr["conv_ms"] * 1e-3) / 1e12
    evals = world * wc["B"] / (wr["ms"] * 1e-3)
    return {"workload": wc["name"], "batch_per_gpu": wc["B"], "value": evals, "unit": UNIT, "ms_per_step": wr["ms"],
            "tower_tflops": evals / world * flops / 1e12, "flops_per_eval": flops,
            "weights": "libtorch-default init seed 42, random BatchNorm", "input": "device-resident board tensor",
            "roofline": {"kernel": f"conv_wide_kernel ({wc['F']}->{wc['F']}, residual+ReLU)", "bound": "tensor",
                         "achieved": conv_tf, "peak": peaks["bf16_burst"], "unit": "TFLOP/s",
                         "frac": conv_tf / peaks["bf16_burst"],
                         "frac_of_sustained": conv_tf / peaks["bf16_sustained"] if peaks["bf16_sustained"] else None,
                         "us_per_launch": wr["conv_ms"] * 1e3,
                         "flops": "real board cells only; the padded (S+1)^2 grid the kernel computes is not counted"}}


def wide_only(args):
    """Only the wide-tower section, single GPU: one JSON line with its entries."""
    import torch
    from omoknuni_small_b200 import capi
    torch.cuda.set_device(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:0")

    def timed(fn, n, per_iter_flush=True):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for s, e in ev:
            if per_iter_flush:
                flush.zero_()
            s.record()
            fn()
            e.record()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in ev]
    peaks = measured_peaks()
    out = []
    for wc in WIDE_NETS:
        wc = dict(wc, B=args.wide_batch or wc["B"])
        out.append(wide_report(time_wide_net(capi, torch, wc, "cuda:0", 0, 0, flush, timed, max(1, min(args.steps, 5))), 1, peaks))
    assert capi.device_error_code() == 0, "a kernel gave up on a bounded wait"
    print(json.dumps({"wide_towers": out}))


def gpu_arm(args):
    import torch
    from omoknuni_small_b200 import capi
    import ctypes as C

    rank, world, local = replicas.rank_info()
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device(dev))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    capi.lib()                       # fails loudly when the CUDA library is missing
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    peaks = measured_peaks()
    shapes = synth.net_tensor_shapes(NET["board_size"], NET["input_channels"], NET["filters"], NET["blocks"],
                                     NET["policy_size"], NET["policy_head_ch"], NET["value_head_ch"])
    w = synth.make_weights(shapes, seed=42, init="kaiming_normal")
    DT = capi.DTYPE_F16 if args.dtype == "f16" else capi.DTYPE_BF16
    DT_OTHER, other_name = (capi.DTYPE_BF16, "bf16") if DT == capi.DTYPE_F16 else (capi.DTYPE_F16, "f16")
    net = capi.Net(17, 15, NET["blocks"], 64, 225, NET["policy_head_ch"], NET["value_head_ch"], 256, B, local, tower_dtype=DT).load(w)
    games, hist, nh, tm = synth.make_gomoku_games(B, 15, seed=replicas.shard_seed(1000, rank))
    d_hist, d_nh, d_tm = (torch.from_numpy(a).to(dev) for a in (hist, nh, tm))
    d_policy = torch.empty((B, 225), dtype=torch.float32, device=dev)
    d_value = torch.empty(B, dtype=torch.float32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # > 126 MB L2

    def step_resident():
        # encode -> tower -> heads from device-resident move histories (ob200_net_forward_gomoku_device)
        net.forward_gomoku_device(d_hist, d_nh, d_tm, d_policy, d_value, capi.OUT_PROBS)

    def timed(fn, n, per_iter_flush=True):
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for s, e in ev:
            if per_iter_flush:
                flush.zero_()
            s.record()
            fn()
            e.record()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in ev]

    # bring the SM clock up from idle before the warm-up steps (memory fills only, none of the measured work):
    # a short run's first timed steps otherwise see the clock still ramping
    for _ in range(int(os.environ.get("OB200_BENCH_SPINUP", "200"))):
        flush.zero_()
    sampler = ClockSampler(local)
    with sampler:
        # the W warm-up steps run with the clock sampler already started: launching it perturbs the host for a
        # moment, and a host that is late with a launch shows up as idle time inside the first step
        for _ in range(W):
            flush.zero_()
            step_resident()
        torch.cuda.synchronize()
        # ---- headline: K steps, device resident ----
        barrier()
        c0 = capi.counters()["kernel_launches"]
        ms = timed(step_resident, K)
        barrier()
        launches = capi.counters()["kernel_launches"] - c0
        total_ms = float(sum(ms))
        if os.environ.get("OB200_BENCH_VERBOSE"):
            print("per-step ms:", " ".join(f"{m:.3f}" for m in ms), file=sys.stderr)
        # ---- e2e: host buffers through the public call ----
        # inputs and outputs in page-locked host memory, allocated once (as an engine would keep them).  The caller
        # keeps two batches in flight (ob200_net_submit_gomoku / ob200_net_wait): while one batch's 926 KB of results
        # travel back, the next batch's kernels run.  Every step still copies its own inputs in and its own results out.
        pin = [torch.from_numpy(a).pin_memory() for a in (hist, nh, tm)]
        p_hist, p_nh, p_tm = (t_.numpy() for t_ in pin)
        out_bufs = [(torch.empty((B, 225), dtype=torch.float32).pin_memory(), torch.empty(B, dtype=torch.float32).pin_memory())
                    for _ in range(2)]
        outs2 = [(a.numpy(), b.numpy()) for a, b in out_bufs]
        for _ in range(2):
            net.infer_gomoku(p_hist, p_nh, p_tm, out=outs2[0])
        torch.cuda.synchronize()
        flush.zero_()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        pending = []
        for i in range(K):
            if len(pending) == 2:
                net.wait(pending.pop(0))
            pending.append(net.submit_gomoku(p_hist, p_nh, p_tm, outs2[i % 2]))
        for tk in pending:
            net.wait(tk)
        e2e_s = time.perf_counter() - t0
        # the same call one batch at a time (submit + wait back to back), L2 flushed before each
        e2e_sync_s = 0.0
        for _ in range(K):
            flush.zero_()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            net.infer_gomoku(p_hist, p_nh, p_tm, out=outs2[0])
            e2e_sync_s += time.perf_counter() - t0
        # ---- the dominant kernel alone: the whole tower (one launch) ----
        bt_in = capi.encode_gomoku(d_hist, d_nh, d_tm, 15, 17, net.input_tensor_channels(), DT)

        # the encoder as a launch of its own (callers that keep their own network; the network step above does not
        # launch it: the tower writes its input planes itself)
        def enc_loop():
            for _ in range(5):
                capi.encode_gomoku(d_hist, d_nh, d_tm, 15, 17, net.input_tensor_channels(), DT, out=bt_in)
        enc_ms = float(np.mean(timed(enc_loop, 3))) / 5
        tower_reps = 5

        def tower_loop():
            for _ in range(tower_reps):
                net.tower_device(bt_in, B)
        tower_loop()
        c_t0 = capi.counters()["kernel_launches"]
        tower_ms = float(np.mean(timed(tower_loop, 5))) / tower_reps
        tower_launches = (capi.counters()["kernel_launches"] - c_t0) // (5 * tower_reps)
        tower_path = net.tower_path()     # 2: boards resident in shared memory, 1: cooperative launch, 0: a launch per layer
        # the same launch with the other 16-bit storage type (same instruction, other operand-format bits)
        net_o = capi.Net(17, 15, NET["blocks"], 64, 225, NET["policy_head_ch"], NET["value_head_ch"], 256, B, local,
                         tower_dtype=DT_OTHER).load(w)
        bt_o = capi.encode_gomoku(d_hist, d_nh, d_tm, 15, 17, net_o.input_tensor_channels(), DT_OTHER)

        def tower_loop_o():
            for _ in range(tower_reps):
                net_o.tower_device(bt_o, B)
        tower_loop_o()
        tower_o_ms = float(np.mean(timed(tower_loop_o, 5))) / tower_reps
        net_o.close()
        # ---- the same network at the other batch sizes of the configurations (256: configs[0]; 4096) ----
        sweep = []
        if not args.no_sweep:
            net_sw = capi.Net(17, 15, NET["blocks"], 64, 225, NET["policy_head_ch"], NET["value_head_ch"], 256, 4096, local,
                              tower_dtype=DT).load(w)
            for Bs in (256, 4096):
                _, h_s, n_s, t_s = synth.make_gomoku_games(Bs, 15, seed=replicas.shard_seed(2000 + Bs, rank))
                dhs, dns, dts = (torch.from_numpy(a).to(dev) for a in (h_s, n_s, t_s))
                pol_s = torch.empty((Bs, 225), dtype=torch.float32, device=dev)
                val_s = torch.empty(Bs, dtype=torch.float32, device=dev)

                def step_s():
                    net_sw.forward_gomoku_device(dhs, dns, dts, pol_s, val_s, capi.OUT_PROBS)
                for _ in range(3):
                    step_s()
                step_ms = float(np.mean(timed(step_s, 5)))
                bts_s = capi.encode_gomoku(dhs, dns, dts, 15, 17, net_sw.input_tensor_channels(), DT)

                def tower_s():
                    for _ in range(tower_reps):
                        net_sw.tower_device(bts_s, Bs)
                tower_s()
                sweep.append((Bs, step_ms, float(np.mean(timed(tower_s, 5))) / tower_reps))
            net_sw.close()
        # ---- one layer as its own launch: 64 -> 64 conv with residual + ReLU ----
        rng = np.random.default_rng(0)
        wp = torch.from_numpy(capi.pack_conv3x3(rng.normal(0, 0.04, (64, 64, 3, 3)).astype(np.float32), None, 64, DT).view(np.int16)).to(dev)
        bias = torch.zeros(64, device=dev)
        n_el = int(capi.lib().ob200_board_tensor_bytes(15, B, 64)) // 2
        bufs = [torch.zeros(n_el, dtype=torch.int16, device=dev) for _ in range(3)]
        reps = 20

        def conv_loop():
            for i in range(reps):
                capi.conv3x3(bufs[i % 3], wp, bias, bufs[(i + 2) % 3], B, 15, 64, 64, True, out=bufs[(i + 1) % 3], dtype=DT)
        conv_loop()
        conv_ms = float(np.mean(timed(conv_loop, 5))) / reps
        # ---- batched PUCT selection + virtual loss, 65,536 x 225 ----
        t = synth.make_selection_tree(SEL_NODES, SEL_CHILDREN, seed=replicas.shard_seed(7, rank))
        dt = capi.DeviceTree(t, dev)
        sel = torch.empty(SEL_NODES, dtype=torch.int32, device=dev)

        def sel_pass():
            dt.select(None, 1.5, 3, True, out=sel)
            dt.vl_revert(sel, 3)

        def sel_only():
            dt.select(None, 1.5, 3, True, out=sel)
        for _ in range(3):
            sel_pass()
        # one pass reads 240 MB, more than the 126 MB L2, so passes run back to back unflushed
        sel_reps = 10

        def sel_pass_loop():
            for _ in range(sel_reps):
                sel_pass()

        def sel_only_loop():
            for _ in range(sel_reps):
                sel_only()
        sel_ms = float(np.mean(timed(sel_pass_loop, 5, per_iter_flush=False))) / sel_reps
        selk_ms = float(np.mean(timed(sel_only_loop, 5, per_iter_flush=False))) / sel_reps
        dt.t["VL"].copy_(torch.from_numpy(t["VL"]).to(dev))
        # ---- the same pass over chess-wide rows: 2,048 nodes x 4,672 children (154 MB per pass) ----
        tw = synth.make_selection_tree(SELW_NODES, SELW_CHILDREN, seed=replicas.shard_seed(9, rank))
        dtw = capi.DeviceTree(tw, dev)
        selw = torch.empty(SELW_NODES, dtype=torch.int32, device=dev)

        def selw_loop():
            for _ in range(5):
                dtw.select(None, 1.5, 3, True, out=selw)
                dtw.vl_revert(selw, 3)
        selw_loop()
        selw_ms = float(np.mean(timed(selw_loop, 3, per_iter_flush=False))) / 5
        del dtw
        # the same rows four times over (8,192 nodes, 617 MB per pass): the 2,048-node pass is a 35 us launch of which
        # about 8 us are ramp-up and tail; this one shows the kernels' steady rate
        tw4 = {k: (np.concatenate([v] * 4) if isinstance(v, np.ndarray) else v) for k, v in tw.items()}
        dtw = capi.DeviceTree(tw4, dev)
        selw = torch.empty(4 * SELW_NODES, dtype=torch.int32, device=dev)
        selw_loop()
        selw_big_ms = float(np.mean(timed(selw_loop, 3, per_iter_flush=False))) / 5
        del dtw, tw, tw4
        # ---- leaf-parallel MCTS: 64 games, 800 simulations per move, leaf batch = B ----
        n_trees, sims = 64, 800
        openings, _, _, _ = synth.make_gomoku_games(n_trees, 15, seed=replicas.shard_seed(100, rank), max_moves=20)
        search = capi.Search(net, n_trees=n_trees, sims_per_move=sims, leaf_batch=B, max_depth=64, c_puct=1.5,
                             virtual_loss=3, dirichlet_alpha=0.3, dirichlet_epsilon=0.25, value_sign=1,
                             transposition_table=True, seed=rank)
        search.run(openings)                                   # warm-up move
        mcts_ms, mcts_wall_ms, mcts_sims, mcts_evals, mcts_moves = 0.0, 0.0, 0, 0, max(2, min(K, 5))
        for _ in range(mcts_moves):
            flush.zero_()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            _, _, st = search.run(openings)
            mcts_wall_ms += (time.perf_counter() - t0) * 1e3          # the whole call as the caller sees it
            mcts_ms += st["device_ms"]; mcts_sims += st["simulations"]; mcts_evals += st["evaluations"]
            mcts_nodes = st["nodes"]
        torch.cuda.synchronize()
        # one more move, outside the figures above, with events around the five phases of every round
        search.phase_timing(True)
        search.run(openings)
        mcts_phases = search.phase_timing(False)
        search.close()
        # ---- the wider towers (parity-test configurations timed for their roofline): Go 19x19 20x128 at
        # batch 2048, chess 8x8 20x256 with 73 policy planes at batch 4096; forward on a resident input ----
        wide = []
        for wc in WIDE_NETS:
            wide.append(time_wide_net(capi, torch, wc, dev, local, rank, flush, timed, min(K, 5)))
    assert capi.device_error_code() == 0, "a kernel gave up on a bounded wait"
    # ---- parity on every rank, after the timed regions: this rank's shard of selection inputs (225-wide and
    # chess-wide rows) and of Gomoku positions against the CPU restatement, bit for bit ----
    from oracle import capi as oc
    sel_ok, enc_ok = 1, 1
    for nodes, children, seed in ((4096, SEL_CHILDREN, 7), (256, SELW_CHILDREN, 9)):
        tp = synth.make_selection_tree(nodes, children, seed=replicas.shard_seed(seed, rank))
        ref = synth.copy_tree(tp)
        dtp = capi.DeviceTree(tp, dev)
        got = dtp.select(None, 1.5, 3, True).cpu().numpy()
        want = oc.puct_select(ref, c_puct=1.5, vl_value=3, apply_vl=True)
        ok = np.array_equal(got, want) and np.array_equal(dtp.host("VL"), ref["VL"])
        dtp.vl_revert(torch.from_numpy(got).to(dev), 3)
        oc.vl_revert(ref, want, 3)
        sel_ok &= int(ok and np.array_equal(dtp.host("VL"), ref["VL"]) and np.array_equal(ref["VL"], tp["VL"]))
    _, h_p, n_p, t_p = synth.make_gomoku_games(256, 15, seed=replicas.shard_seed(1000, rank))
    for dt_enc in (capi.DTYPE_BF16, capi.DTYPE_F16):
        bt_p = capi.encode_gomoku(torch.from_numpy(h_p).to(dev), torch.from_numpy(n_p).to(dev), torch.from_numpy(t_p).to(dev), 15, 19, 64, dt_enc)
        torch.cuda.synchronize()
        planes_p, pad_zero = capi.board_tensor_to_planes(bt_p.cpu().numpy().view(np.uint16), 15, 256, 64, dt_enc)
        enc_ok &= int(pad_zero and np.array_equal(planes_p[:, :19], oc.gomoku_encode(h_p, n_p, t_p, 15, 19)) and not planes_p[:, 19:].any())
    parity = replicas.sum_counters(dist, {"selection_ranks_ok": sel_ok, "encode_ranks_ok": enc_ok}, dev)

    reduced = replicas.max_over_ranks(
        dist, [total_ms, e2e_s * 1e3, conv_ms, sel_ms, selk_ms, mcts_ms, selw_ms, tower_ms, tower_o_ms, e2e_sync_s * 1e3, mcts_wall_ms, selw_big_ms, enc_ms] + [v for _, m, tm in sweep for v in (m, tm)] + [v for wr in wide for v in (wr["ms"], wr["conv_ms"])], dev)
    total_ms, e2e_ms, conv_ms, sel_ms, selk_ms, mcts_ms, selw_ms, tower_ms, tower_o_ms, e2e_sync_ms, mcts_wall_ms, selw_big_ms, enc_ms = reduced[:13]
    sweep = [(bs, reduced[13 + 2 * i], reduced[14 + 2 * i]) for i, (bs, _, _) in enumerate(sweep)]
    for i, wr in enumerate(wide):
        wr["ms"], wr["conv_ms"] = reduced[13 + 2 * len(sweep) + 2 * i], reduced[14 + 2 * len(sweep) + 2 * i]
    totals = replicas.sum_counters(dist, capi.counters(), dev)   # the only cross-GPU step: per-GPU counters summed
    if rank == 0:
        flops_eval = synth.net_flops_per_eval(15, 17, 64, NET["blocks"], 225, NET["policy_head_ch"], NET["value_head_ch"])
        value = replicas.aggregate_throughput(B, K, world, total_ms)
        conv_flops = 2.0 * 225 * 9 * 64 * 64 * B
        conv_tf = conv_flops / (conv_ms * 1e-3) / 1e12
        tower_flops = (2.0 * 225 * 9 * 17 * 64 + NET["blocks"] * 2 * 2.0 * 225 * 9 * 64 * 64) * B
        tower_tf = tower_flops / (tower_ms * 1e-3) / 1e12
        sel_bytes = synth.selection_bytes_per_node(SEL_CHILDREN) * SEL_NODES
        selk_bytes = sel_bytes - 16 * SEL_NODES      # the select kernel alone: without the revert's read-modify-write
        clocks = sampler.summary()
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": args.dtype, "data": "synthetic",
            "config": arm_config(B, world),
            "e2e": {"value": world * B * K / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": B * 34,
                    "d2h_bytes_per_step": B * 226 * 4,
                    "how": "ob200_net_submit_gomoku / ob200_net_wait with two batches in flight, pinned host buffers, wall clock over all steps; every batch's inputs come from host memory and its results go back there, L2 flushed once before the first batch (one_batch_at_a_time: before every batch)",
                    "one_batch_at_a_time": world * B * K / (e2e_sync_ms * 1e-3)},
            "gpu_launches": int(launches), "counters_all_gpus": totals,
            "tower_tflops": value / world * flops_eval / 1e12,
            "roofline": {"kernel": {2: "conv_tower_resident_kernel (stem + 20 convolutions 64->64 in one launch, boards resident in shared memory)",
                                    1: "conv_tower_kernel (stem + 20 convolutions 64->64 in one cooperative launch)",
                                    0: "conv3x3_kernel x 21 (one launch per layer)"}.get(tower_path, "?"),
                         "bound": "tensor", "achieved": tower_tf, "peak": peaks["bf16_burst"], "unit": "TFLOP/s",
                         "frac": tower_tf / peaks["bf16_burst"],
                         "frac_of_sustained": tower_tf / peaks["bf16_sustained"] if peaks["bf16_sustained"] else None,
                         "peak_source": peaks["source"] + " (burst: kernel timed alone)", "us_per_launch": tower_ms * 1e3,
                         "launches_per_tower": int(tower_launches), "flops_per_launch": tower_flops,
                         # DRAM bytes per launch from the ncu captures at batch 512, scaled by the boards processed: the
                         # input tensor and the weights are read; the board-resident tower writes nothing back to DRAM
                         # (its output stays in L2), the cooperative-launch tower works out of L2 after the first layer
                         "traffic": {2: 18.38e6, 1: 21.05e6}.get(tower_path, 21 * 33.66e6) * B / 512.0, "traffic_unit": "bytes/launch",
                         # the same kernel as the network step launches it (input planes written from the move histories,
                         # no input tensor): the packed weights once and 34 bytes of history per board
                         "traffic_in_step": 1.765e6 + 34.0 * B,
                         "traffic_source": {2: "profiles/conv_tower_resident_kernel_gomoku15_batch512.md (scaled by batch)",
                                            1: "profiles/conv_tower_kernel_gomoku15_batch512.md (scaled by batch)"}.get(
                                                tower_path, "profiles/conv3x3_kernel_gomoku15_batch512.md (21 launches, scaled by batch)")},
            # the tower launch with the other 16-bit storage type: same tcgen05.mma rate, so the same fraction is expected
            "roofline_" + other_name: {"us_per_launch": tower_o_ms * 1e3, "achieved": tower_flops / (tower_o_ms * 1e-3) / 1e12,
                                       "unit": "TFLOP/s", "frac": tower_flops / (tower_o_ms * 1e-3) / 1e12 / peaks["bf16_burst"],
                                       "note": "identical launch, tower weights and board tensors stored as " + other_name},
            "roofline_conv_layer": {"kernel": "conv3x3_kernel (64->64, residual+ReLU), one layer as its own launch",
                         "bound": "tensor", "achieved": conv_tf,
                         "peak": peaks["bf16_burst"], "unit": "TFLOP/s", "frac": conv_tf / peaks["bf16_burst"],
                         "frac_of_sustained": conv_tf / peaks["bf16_sustained"] if peaks["bf16_sustained"] else None,
                         "peak_source": peaks["source"] + " (burst: kernel timed alone)", "us_per_launch": conv_ms * 1e3,
                         # DRAM bytes per launch from the ncu capture at batch 512 (cold cache: input +
                         # residual from DRAM, output left in L2), scaled by the boards processed
                         "traffic": 33.66e6 * B / 512.0, "traffic_unit": "bytes/launch",
                         "traffic_source": "profiles/conv3x3_kernel_gomoku15_batch512.md (scaled by batch)"},
            # the stand-alone encoder launch: 8 KB of 17-plane positions per board (225 x 17 x 2 B + 34 B of history in) by the
            # north star's count; the kernel writes the whole padded 64-channel board tensor (32 KB per board)
            "encoder": {"kernel": "encode_gomoku_board_kernel", "us_per_launch": enc_ms * 1e3, "boards": B,
                        "algorithmic_gbs": B * (225 * 17 * 2 + 34) / (enc_ms * 1e-3) / 1e9,
                        "written_gbs": B * 256 * 64 * 2 / (enc_ms * 1e-3) / 1e9,
                        "note": "not part of the network step: the tower writes its own input planes"},
            "selection": {"value": SEL_NODES / (sel_ms * 1e-3), "unit": "node selections/s (select + VL apply + VL revert)",
                          "nodes": SEL_NODES, "children": SEL_CHILDREN, "ms_per_pass": sel_ms,
                          # the whole pass (select + apply, then the clamped revert): 3,656 algorithmic bytes per node
                          "pass_roofline": {"bound": "hbm", "achieved": sel_bytes / (sel_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                            "frac": sel_bytes / (sel_ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "us_per_pass": sel_ms * 1e3,
                                            "algorithmic_bytes": sel_bytes, "peak_source": peaks["source"]},
                          # the select + apply kernel alone
                          "roofline": {"kernel": "puct_select_staged_kernel", "bound": "hbm",
                                       "achieved": selk_bytes / (selk_ms * 1e-3) / 1e9, "peak": peaks["hbm_gbs"],
                                       "unit": "GB/s", "frac": selk_bytes / (selk_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                       "peak_source": peaks["source"], "us_per_launch": selk_ms * 1e3,
                                       "algorithmic_bytes": selk_bytes, "traffic": 246.8e6, "traffic_unit": "bytes/launch",
                                       "traffic_source": "profiles/puct_select_staged_kernel_65536x225.md"},
                          "pass_gbs": sel_bytes / (sel_ms * 1e-3) / 1e9,
                          "wide_rows": {"nodes": SELW_NODES, "children": SELW_CHILDREN, "ms_per_pass": selw_ms,
                                        "value": SELW_NODES / (selw_ms * 1e-3), "unit": "node selections/s (select + VL apply + VL revert)",
                                        "kernel": "puct_select_segmented_kernel (256-slot segments through per-warp rings) + puct_select_finish_kernel",
                                        "achieved_gbs": synth.selection_bytes_per_node(SELW_CHILDREN) * SELW_NODES / (selw_ms * 1e-3) / 1e9,
                                        "frac_of_hbm": synth.selection_bytes_per_node(SELW_CHILDREN) * SELW_NODES / (selw_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
                                        # the same pass over four times the nodes (617 MB): the kernels' steady rate
                                        "at_8192_nodes": {"ms_per_pass": selw_big_ms,
                                                          "achieved_gbs": synth.selection_bytes_per_node(SELW_CHILDREN) * 4 * SELW_NODES / (selw_big_ms * 1e-3) / 1e9,
                                                          "frac_of_hbm": synth.selection_bytes_per_node(SELW_CHILDREN) * 4 * SELW_NODES / (selw_big_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}}},
            "mcts": {"value": world * mcts_sims / (mcts_ms * 1e-3), "unit": "simulations/s",
                     # the same simulations over the wall clock around ob200_search_run (root set-up, noise sampling,
                     # copies, the wait and the read-back of the visit counts included)
                     "wall_value": world * mcts_sims / (mcts_wall_ms * 1e-3), "ms_per_move_wall": mcts_wall_ms / mcts_moves,
                     "leaf_evals_per_sec": world * mcts_evals / (mcts_ms * 1e-3),
                     "config": {"games_per_gpu": 64, "sims_per_move": 800, "leaf_batch": B, "c_puct": 1.5, "virtual_loss": 3,
                                "dirichlet": [0.3, 0.25], "openings": "seeded random, 0-20 stones", "moves_timed": mcts_moves,
                                "transposition_table": "on (device table, Zobrist keys)", "nodes_per_move": mcts_nodes},
                     "ms_per_move": mcts_ms / mcts_moves,
                     # rank 0's phase sums over one extra move timed with events between the phases (which costs the
                     # overlap of each phase's launch with its predecessor, so the sum exceeds ms_per_move); the descent
                     # reads a row of 3,656 B per tree level, the network is the step above
                     "phases_ms_one_move": mcts_phases,
                     "timing": "value: CUDA events around the enqueued work of each move, inside the library; wall_value: perf_counter around the call"},
            "batch_sweep": [{"leaf_batch_per_gpu": bs, "ms_per_step": m, "value": world * bs / (m * 1e-3), "unit": UNIT,
                             "tower_tflops": bs / (m * 1e-3) * flops_eval / 1e12,
                             # the tower launch alone at this batch, as in `roofline`
                             "tower_launch": {"us_per_launch": tm * 1e3, "achieved": tower_flops / B * bs / (tm * 1e-3) / 1e12,
                                              "unit": "TFLOP/s", "frac": tower_flops / B * bs / (tm * 1e-3) / 1e12 / peaks["bf16_burst"]}}
                            for bs, m, tm in sweep],
            "wide_towers": [wide_report(wr, world, peaks) for wr in wide],
            "clocks": clocks,
            # ranks whose selection (indices and virtual-loss state after apply and after revert; 4,096 x 225 and
            # 256 x 4,672 rows of the rank's own shard) and Gomoku encoding (256 positions, both storage types) equal
            # the CPU restatement bit for bit
            "parity": dict(parity, ranks=world),
        }
        if world == 1 and not args.no_cpu:
            base, _ = cpu_baseline(3, 1)
            line["cpu_baseline"] = base
            line["selection"]["cpu_baseline"] = selection_cpu_baseline()
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if parity["selection_ranks_ok"] != world or parity["encode_ranks_ok"] != world:
        print(f"parity mismatch: {parity} of {world} ranks", file=sys.stderr)
        sys.exit(1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=1024, help="leaf batch per GPU")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--dtype", default="f16", choices=["f16", "bf16"],
                    help="storage type of the tower's weights and activations (fp32 accumulate either way); fp16 is what "
                         "holds the 2e-2 / 1e-2 tolerance against the fp32 forward on the benchmark's weights")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch 256 / 4096 runs of the same network")
    ap.add_argument("--wide-only", action="store_true",
                    help="time only the Go / chess towers (a short run for profiling; not the contract line)")
    ap.add_argument("--wide-batch", type=int, default=0, help="with --wide-only: batch for both towers")
    args = ap.parse_args()
    # stdout carries the one JSON line and nothing else: while the benchmark runs, file descriptor 1
    # points at stderr (libraries such as NCCL print banners with printf), and print() is given the
    # real stdout back only for the result line
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    result = io.StringIO()
    try:
        with contextlib.redirect_stdout(result):
            if args.impl == "reference":
                reference_arm(args)
            elif args.wide_only:
                wide_only(args)
            else:
                gpu_arm(args)
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        os.close(real_stdout)
    out = result.getvalue()
    if out:
        sys.stdout.write(out)
        sys.stdout.flush()


if __name__ == "__main__":
    main()
