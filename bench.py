"""Benchmark of the quantized-expert decode path (one JSON line on stdout).

Workload (N = 1): one decode step of a stack of MoE layers, each with 512 IQ3_S experts
(hidden 2560, intermediate 512, gate/up/down all IQ3_S), a bf16 router ~ N(0, 0.02), softmax top-10
routing, batch 16 tokens of fp32 x ~ N(0, 1) per layer. The layers only rotate the weight set: every
layer owns its own 865 MB of expert bytes, so with >= 8 layers each launch streams weights the
126 MB L2 cannot hold. metric = weight bytes the step has to read (distinct routed experts x
1,689,600 B + router) / device time, in GB/s.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

--impl reference times the reference's own CPU expert path (oracle/_ref when it was built and the
host CPU can run it, else this repository's scalar restatement) on the host cores, same metric.
N > 1 (launched under torchrun, one rank per GPU) shards the 512 experts over the ranks; see
fngine_b200/ep.py.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FMT = 21  # IQ3_S
INTER = 512
HIDDEN = 2560
TOPK = 10
EXPERTS = 512
BLOB = 1689600
ROUTER_BYTES = EXPERTS * HIDDEN * 2


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        for r in self.rows:
            if len(r) < 9:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def host_routing(wr_bits, x):
    """Router projection and top-10 on the host (numpy fp32 + the oracle's top-k)."""
    from fngine_b200 import synth
    from oracle import oracle as O
    logits = x.astype(np.float32) @ synth.bf16_bits_to_f32(wr_bits).T
    return O.topk(np.ascontiguousarray(logits[:, :EXPERTS]))


def cpu_layer_runner(seed, x, ids, w, threads):
    """Returns (callable running one CPU MoE layer step, bytes it streams, kind)."""
    from fngine_b200 import synth
    from oracle import oracle as O
    lib = O.ref()
    kind = "reference" if lib is not None else "port"
    used = sorted(set(ids.reshape(-1).tolist()))
    tables = {FMT: synth.d_table(FMT)}
    blobs = np.concatenate([synth.expert_blob(FMT, FMT, INTER, seed, e, tables=tables) for e in used])
    ids2 = np.vectorize({e: i for i, e in enumerate(used)}.get)(ids).astype(np.int32)

    def run():
        return O.moe_layer(FMT, FMT, HIDDEN, INTER, blobs, BLOB, x, ids2, w, threads=threads, lib=lib)

    return run, len(used) * BLOB + ROUTER_BYTES, kind


def run_reference(args, rank):
    """The reference arm: the reference's CPU expert path on the host cores, rank 0 only."""
    if rank != 0:
        return
    from fngine_b200 import synth
    threads = os.cpu_count() or 1
    layers = min(args.layers, 4)
    runners = []
    for l in range(layers):
        wr = synth.router_weights(9000 + l)
        x = synth.activations(7000 + l, args.batch)
        ids, w = host_routing(wr, x)
        runners.append(cpu_layer_runner(5000 + l, x, ids, w, threads))
    kind = runners[0][2]
    for i in range(args.warmup):
        runners[i % layers][0]()
    t0 = time.perf_counter()
    nbytes = 0
    for i in range(args.steps):
        run, b, _ = runners[i % layers]
        run()
        nbytes += b
    dt = time.perf_counter() - t0
    gbs = nbytes / dt / 1e9
    sample = ("%d steps, each ONE MoE layer of batch %d (distinct routed experts only) out of the %d layers a full "
              "step has, %d layers rotated" % (args.steps, args.batch, args.layers, layers))
    line = {"impl": "reference", "metric": "iq3s_expert_gemv_hbm_gbs", "value": gbs, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": workload_config(args, args.layers),
            "tokens_per_s": args.batch * args.steps / dt,
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def workload_config(args, layers_per_step):
    return {"workload": "MoE layer at decode: 512 IQ3_S experts (hidden 2560, inter 512, gate/up/down IQ3_S), "
                        "bf16 router N(0,0.02), softmax top-10, batch %d fp32 x~N(0,1)" % args.batch,
            "batch": args.batch, "layers_per_step": layers_per_step, "experts": EXPERTS, "top_k": TOPK,
            "l2_policy": "inputs larger than L2: every layer has its own 865 MB expert set, "
                         "%d layers rotate (%.1f GB resident)" % (args.layers, args.layers * EXPERTS * BLOB / 1e9),
            "activation_format": "Q8_K (reference CPU tier numerics)"}


# DRAM bytes moved / algorithmic bytes of one launch of the expert kernel (gate/up + down of every routed
# expert), from an ncu capture of layer 0 of the benchmark workload (139 experts: 235.05 MB read + 4.24 MB
# written for 234.85 MB of expert bytes): traffic grows with the expert count like the algorithmic bytes do, so
# the ratio carries over to the other layers.
EXPERTS_DRAM_TRAFFIC_RATIO = 239.30 / 234.85


def single_expert_section(torch, layers, routers, steps):
    """One token through ONE routed expert per layer (the single-expert case the benchmark definition opens
    with), on the GPU: the decode layer call with a slot map that holds only the token's best expert (the
    other nine count as experts of another rank), CUDA-graph replays over the rotating layers, so the
    1,689,600 weight bytes of every call come from HBM. Three launches per call (route, experts, combine)."""
    import types
    from fngine_b200 import ep, moe, synth
    ws = moe.DecodeWorkspace(layers[0])
    n = len(layers)
    xs = [torch.from_numpy(synth.activations(7300 + l, 1)).cuda() for l in range(n)]
    y = torch.empty(1, HIDDEN, dtype=torch.float32, device="cuda")
    shards = []
    for l in range(n):
        moe.moe_layer_decode(routers[l], layers[l], xs[l], ws, y)
        torch.cuda.synchronize()
        best = int(ws.work().topk_expert[0][0])
        slot_of = np.full(EXPERTS, -1, dtype=np.int32)
        slot_of[best] = best
        shards.append(types.SimpleNamespace(layer=layers[l], slot_of=torch.from_numpy(slot_of).cuda()))
    g = torch.cuda.CUDAGraph()
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        for l in range(n):
            ep.layer_decode_ep(routers[l], shards[l], xs[l], ws, y)
        with torch.cuda.graph(g, stream=st):
            for l in range(n):
                ep.layer_decode_ep(routers[l], shards[l], xs[l], ws, y)
    torch.cuda.synchronize()
    items = ws.work().n_items
    for _ in range(3):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) / steps / n * 1e3
    return {"us_per_call": us, "experts_per_call": items, "weight_bytes_per_call": BLOB,
            "gbs": (BLOB + ROUTER_BYTES) / us / 1e3, "timing": "CUDA graph of %d rotating layers" % n,
            "call": "fb_moe_layer_decode_ep with one resident expert of the token's ten", "device_status": ws.status()}


def iq4nl_section(torch, steps, n_layers=4, fg=20, fd=20, inter=INTER, batches=(1, 8)):
    """The IQ4_NL resident-expert variant (18-byte blocks, Q8_0 activations): the same decode layer at batch
    1 and 8, four rotating layers (4.5 GB, larger than L2), CUDA-graph replays, device time. With other
    formats: the same measurement for a layer of the reference's other expert formats (plain kernels)."""
    from fngine_b200 import moe, synth
    blob = synth.blob_bytes(fg, fd, inter)
    layers = [moe.synth_layer(fg, fd, inter, EXPERTS, 6000 + l) for l in range(n_layers)]
    routers = [torch.from_numpy(synth.router_weights(9100 + l).view(np.int16)).cuda().view(torch.bfloat16)
               for l in range(n_layers)]
    ws = moe.DecodeWorkspace(layers[0])
    res = {}
    for b in batches:
        xs = [torch.from_numpy(synth.activations(7100 + l, b)).cuda() for l in range(n_layers)]
        y = torch.empty(b, HIDDEN, dtype=torch.float32, device="cuda")
        d = []
        for l in range(n_layers):
            moe.moe_layer_decode(routers[l], layers[l], xs[l], ws, y)
            torch.cuda.synchronize()
            d.append(ws.work().n_items)
        g = torch.cuda.CUDAGraph()
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for l in range(n_layers):
                    moe.moe_layer_decode(routers[l], layers[l], xs[l], ws, y)
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = e0.elapsed_time(e1) / steps
        by = sum(k * blob + ROUTER_BYTES for k in d)
        res[str(b)] = {"gbs": by / t / 1e6, "us_per_layer": t / n_layers * 1e3, "distinct_experts_mean": sum(d) / n_layers}
    if (fg, fd, inter) == (20, 20, INTER):
        res["workload"] = "512 IQ4_NL experts per layer (2,211,840 B each), Q8_0 activations, %d rotating layers" % n_layers
    else:
        res["workload"] = "512 experts per layer, gate/up ggml type %d, down type %d, intermediate %d (%d B each), %d " \
                          "rotating layers; plain (untuned) kernels for the formats beside IQ3_S and IQ4_NL" % (fg, fd, inter, blob, n_layers)
    res["device_status"] = ws.status()
    del layers
    torch.cuda.empty_cache()
    return res


def fp8_gemm_section(torch, iters=10):
    """The FP8-row dense GEMM of the benchmark definition (bf16 [4096x2560] x E4M3 [9216x2560] -> bf16), both
    activation routes, each call timed alone with CUDA events after an L2 flush; the library FP8 GEMM of the
    same shape (torch._scaled_mm, when present) gives the practical tensor-core ceiling on this box.
    rel_u = relative L2 error against the fp32 reference on dequantized weights and the given bf16
    activations (the stated 2e-2 bar); rel_q (A8 only) = against the same reference fed A8's own
    per-token E4M3 activations."""
    from fngine_b200 import lib as L
    from fngine_b200 import linear, synth
    from oracle import oracle as O
    T, N, K = 4096, 9216, 2560
    codes, scales = synth.fp8_row_weight(4, N, K)
    wc, ws = torch.from_numpy(codes).cuda(), torch.from_numpy(scales).cuda()
    weight = linear.Fp8RowWeight(wc, ws)
    x = torch.from_numpy(synth.to_bf16_bits(synth.activations(44, T, hidden=K)).view(np.int16)).cuda().view(torch.bfloat16)
    out = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
    work = linear.linear_fp8_workspace(weight, T)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    xq, xs = linear.fp8_quantize_tokens(x)

    def timed(fn):
        ts = []
        for _ in range(3):
            fn()
        for _ in range(iters):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        return statistics.median(ts), min(ts)

    flops = 2.0 * T * N * K
    tab = torch.from_numpy(O.e4m3_table()).cuda()  # the checker: outside every timed region
    wd = tab[wc.long()] * ws[:, None]
    ref_u = x.float() @ wd.T
    res = {"shape": "bf16[4096x2560] x e4m3[9216x2560] -> bf16[4096x9216], fp32 row scales",
           "nominal_dense_fp8_tflops": 4500.0, "l2_policy": "256 MB flush write before every timed call",
           "flop_count": "2 x 4096 x 9216 x 2560 for both routes (the exact route issues twice the tensor-core work)"}
    peaks_json = os.path.join(ROOT, "MEASURED_PEAKS.json")
    bf16_burst = float(json.load(open(peaks_json))["bf16_tflops"]) if os.path.exists(peaks_json) else 1590.0
    for name, path in (("exact", L.FP8_PATH_AUTO), ("a8", L.FP8_PATH_A8)):
        med, best = timed(lambda: linear.linear_fp8(x, weight, out, work, path=path))
        linear.linear_fp8(x, weight, out, work, path=path)
        torch.cuda.synchronize()
        got = out.float()
        tf = flops / (med * 1e-3) / 1e12
        entry = {"tflops": tf, "tflops_best": flops / (best * 1e-3) / 1e12, "ms": med,
                 "frac_of_nominal_fp8": tf / 4500.0, "frac_of_measured_bf16_burst": tf / bf16_burst,
                 "rel_u": float((got - ref_u).norm() / ref_u.norm()),
                 "includes": "activation pieces kernel + tcgen05 GEMM + scale/bf16 epilogue"}
        if name == "a8":
            ref_q = (tab[xq.long()] * xs[:, None]) @ wd.T
            entry["rel_q"] = float((got - ref_q).norm() / ref_q.norm())
            entry["route"] = "Fp8LinearPath::A8: one E4M3 code per activation, per-token scale max|x|/448 (on request only)"
        else:
            entry["route"] = ("Fp8LinearPath::Auto / A16: bf16 activations kept exactly as two E4M3 pieces, two MMAs per "
                              "K step into one accumulator (meets the stated 2e-2 bar)")
        res[name] = entry
    try:
        a8 = xq.view(torch.float8_e4m3fn)
        b8 = wc.view(torch.float8_e4m3fn).t()
        one = torch.ones((), dtype=torch.float32, device="cuda")
        lm, lb = timed(lambda: torch._scaled_mm(a8, b8, scale_a=one, scale_b=one, out_dtype=torch.bfloat16))
        res["library_fp8_gemm_tflops"] = flops / (lm * 1e-3) / 1e12
        res["a8"]["frac_of_library"] = lm / res["a8"]["ms"]
        xb = x
        wb = wd.to(torch.bfloat16).t().contiguous()
        bm, _ = timed(lambda: torch.matmul(xb, wb))
        res["library_bf16_gemm_tflops"] = flops / (bm * 1e-3) / 1e12
        res["exact"]["frac_of_library_bf16"] = bm / res["exact"]["ms"]
    except Exception as e:  # the comparison is optional
        res["library_fp8_gemm_tflops"] = None
        res["library_note"] = type(e).__name__
    return res


def fp8_decode_section(torch, iters=10):
    """Decode-width FP8-row projections (T <= 16, exact bf16 activations): the dense shapes of one decode step
    that the reference registers (src/kernels/linear/linear.h:8-18), each call (activation split + streaming
    kernel) timed alone with CUDA events after an L2 flush. Bytes = weight codes + row scales."""
    from fngine_b200 import linear
    peak, _ = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(5)
    res = {"l2_policy": "256 MB flush write before every call",
           "timing": "CUDA graph of %d x (flush, call) minus a graph of %d x flush, CUDA events around the replays, "
                     "median of 5 (a call timed eagerly is bounded by its host-side launch work, about 20 us)" % (iters, iters),
           "shapes": {}}

    def graph_time(fn):
        for _ in range(3):
            flush.fill_(1)
            fn()
        torch.cuda.synchronize()

        def build(with_call):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(iters):
                    flush.fill_(1)
                    if with_call:
                        fn()
            return g

        def run(g):
            ts = []
            g.replay()
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                g.replay()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            return statistics.median(ts)

        return (run(build(True)) - run(build(False))) / iters

    shapes = [("gdn.qkvz", 16384, 2560, "store_bf16"), ("gdn.out", 2560, 6144, "gr_write"),
              ("moe.shared_gate_up", 1280, 2560, "swiglu"), ("moe.shared_down", 2560, 640, "shared_scale"),
              ("lm_head", 248320, 2560, "store_f32")]
    for name, n, k, kind in shapes:
        mag = torch.randint(0, 0x78, (n, k), dtype=torch.uint8, device="cuda", generator=gen)
        sign = torch.randint(0, 2, (n, k), dtype=torch.uint8, device="cuda", generator=gen) << 7
        weight = linear.Fp8RowWeight(mag | sign, (torch.rand(n, device="cuda", generator=gen) * 1e-3 + 1e-4).to(torch.bfloat16))
        del mag, sign
        work = linear.linear_fp8_decode_workspace(weight)
        entry = {}
        for T in (1, 16):
            x = torch.randn(T, k, device="cuda", generator=gen).to(torch.bfloat16)
            if kind == "store_bf16":
                epi = linear.store_bf16(torch.empty(T, n, dtype=torch.bfloat16, device="cuda"))
            elif kind == "store_f32":
                epi = linear.store_f32(torch.empty(T, n, dtype=torch.float32, device="cuda"))
            elif kind == "swiglu":
                epi = linear.swiglu(torch.empty(T, n // 2, dtype=torch.bfloat16, device="cuda"))
            elif kind == "shared_scale":
                logit = torch.randn(T, 513, device="cuda", generator=gen)
                epi = linear.shared_scale(torch.empty(T, n, dtype=torch.float32, device="cuda"), logit[:, 512:], 513)
            else:
                inj = torch.randn(T, 4, device="cuda", generator=gen)
                epi = linear.gr_write(torch.zeros(T, 4, n, device="cuda"), inj)
            med = graph_time(lambda: linear.linear_fp8_decode(x, weight, epi, work))
            gbs = (n * k + 2 * n) / (med * 1e-3) / 1e9
            entry["T%d" % T] = {"us": med * 1e3, "gbs": gbs, "frac_of_hbm_peak": gbs / peak}
        res["shapes"]["%s %dx%d %s" % (name, n, k, kind)] = entry
        del weight, work
        torch.cuda.empty_cache()
    return res


def legacy_section(torch, n_layers=4, steps=20):
    """The reference's own GPU decode kernels (src/kernels/moe/moe_decode.cu, compiled unchanged for sm_100a
    into oracle/_ref_gpu by oracle/build_ref_gpu.py: test infrastructure, never on the product path) beside this
    library's, on this GPU, at the reference's native shape: 512 experts per layer with IQ3_S gate/up [640 x 2560]
    and IQ4_NL down [2560 x 640] (2,329,600 B each), bf16 tokens, T = 1, 4, 9. Both sides run the reference's
    four-call decode sequence (select -> hot gate/up -> hot down -> combine with the residual write) from the same
    router logits, as CUDA-graph replays over rotating layers (4.8 GB, larger than L2). The two differ in
    activation numerics (the reference GPU tier quantizes per 32 values with an fp32 scale, this library follows
    the CPU tier's Q8_K / Q8_0), so their results agree to the ~1e-2 those two families have between themselves."""
    import ctypes
    from fngine_b200 import moe, synth
    so = os.path.join(ROOT, "oracle", "_ref_gpu", "libfngine_ref_gpu.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref_gpu is not built (needs the reference checkout at build time)"}
    ref = ctypes.CDLL(so)
    ref.refgpu_decode_workspace_bytes.restype = ctypes.c_size_t
    ref.refgpu_layer_decode.restype = ctypes.c_int
    ref.refgpu_layer_decode.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fg, fd, inter = 21, 20, 640
    blob = synth.blob_bytes(fg, fd, inter)
    layers = [moe.synth_layer(fg, fd, inter, EXPERTS, 8000 + l) for l in range(n_layers)]
    routers = [torch.from_numpy(synth.router_weights(9200 + l, rows=513).view(np.int16)).cuda().view(torch.bfloat16)
               for l in range(n_layers)]
    ws = moe.DecodeWorkspace(layers[0])
    rbuf = torch.zeros(ref.refgpu_decode_workspace_bytes() + 256, dtype=torch.uint8, device="cuda")
    rbase = (rbuf.data_ptr() + 255) & ~255
    res = {"shape": "512 experts/layer, IQ3_S gate/up [640x2560] + IQ4_NL down [2560x640], %d rotating layers" % n_layers,
           "sequence": "select -> hot gate/up -> hot down -> combine (the reference's four decode calls), CUDA graph"}
    for T in (1, 4, 9):
        xs = [torch.from_numpy(synth.to_bf16_bits(synth.activations(7200 + l, T)).view(np.int16)).cuda().view(torch.bfloat16)
              for l in range(n_layers)]
        logits = [torch.empty(T, 513, dtype=torch.float32, device="cuda") for _ in range(n_layers)]
        for l in range(n_layers):
            moe.router_logits(routers[l], xs[l], logits[l])
        zeros = torch.zeros(T, HIDDEN, dtype=torch.float32, device="cuda")
        inj = torch.zeros(T, 4, dtype=torch.float32, device="cuda")
        X = torch.zeros(T, 4, HIDDEN, dtype=torch.float32, device="cuda")
        y_ours = torch.empty(T, HIDDEN, dtype=torch.float32, device="cuda")
        y_ref = torch.empty(T, HIDDEN, dtype=torch.float32, device="cuda")

        def ours(l):
            moe.moe_select_publish(logits[l], xs[l], None, 0, None, None, T, ws)
            moe.moe_hot_gate_up(layers[l], T, ws)
            moe.moe_hot_down(layers[l], T, ws)
            moe.moe_combine(ws, zeros, None, 0, None, inj, X, y_ours, T)

        def theirs(l):
            st = ref.refgpu_layer_decode(logits[l].data_ptr(), xs[l].data_ptr(), layers[l].slots.data_ptr(), blob, fg, fd, T,
                                         rbase, zeros.data_ptr(), inj.data_ptr(), X.data_ptr(), y_ref.data_ptr(),
                                         torch.cuda.current_stream().cuda_stream)
            if st:
                raise RuntimeError("reference decode kernels returned cudaError %d" % st)

        ours(0)
        theirs(0)
        torch.cuda.synchronize()
        diff = float((y_ours - y_ref).norm() / y_ref.norm())
        distinct = ws.work().n_items
        entry = {"rel_l2_between_the_two": diff, "distinct_experts_layer0": distinct}
        for name, fn in (("this_library", ours), ("reference_kernels", theirs)):
            for l in range(n_layers):
                fn(l)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            st = torch.cuda.Stream()
            st.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(st):
                with torch.cuda.graph(g, stream=st):
                    for l in range(n_layers):
                        fn(l)
            torch.cuda.synchronize()
            for _ in range(3):
                g.replay()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            entry[name + "_us_per_layer"] = a.elapsed_time(b) / steps / n_layers * 1e3
        res["T%d" % T] = entry
    res["device_status"] = ws.status()
    del layers
    torch.cuda.empty_cache()
    return res


def prefill_cpu_baseline(seed, x_bits, ids, budget_s=8.0):
    """The reference's CPU prefill path (decode_rows_bf16 + gemm_bf16 per expert, h rounded to bf16) on a
    bounded sample: the first tokens of layer 0 with their real routing, experts spread over the host cores.
    Returns (expert-token pairs per second, pairs done, threads, kind)."""
    from concurrent.futures import ThreadPoolExecutor
    from fngine_b200 import synth
    from oracle import oracle as O
    lib = O.ref()
    kind = "reference" if lib is not None else "port"
    threads = os.cpu_count() or 1
    by_expert = {}
    for t in range(ids.shape[0]):
        for e in ids[t].tolist():
            by_expert.setdefault(int(e), []).append(t)
    tables = {FMT: synth.d_table(FMT)}
    jobs = [(synth.expert_blob(FMT, FMT, INTER, seed, e, tables=tables), np.ascontiguousarray(x_bits[toks]))
            for e, toks in sorted(by_expert.items())]

    def one(job):
        O.expert_ffn_bf16(FMT, FMT, HIDDEN, INTER, job[0], job[1], lib=lib)
        return job[1].shape[0]

    t0 = time.perf_counter()
    done = 0
    with ThreadPoolExecutor(max_workers=threads) as pool:  # ctypes releases the GIL inside the C call
        for lo in range(0, len(jobs), 4 * threads):
            done += sum(pool.map(one, jobs[lo:lo + 4 * threads]))
            if time.perf_counter() - t0 > budget_s:
                break
    return done / (time.perf_counter() - t0), done, threads, kind


def prefill_section(torch, n_layers=48, tokens=8192, steps=2):
    """The 48-layer routed-expert stack at prefill on one GPU: 8192 bf16 tokens, 512 IQ3_S experts per
    layer (inter 512), top-10, router logits = bf16 projection (std 0.02) + a Zipf(1.1) popularity bias
    over a seeded permutation of the experts (bias = -1.1 * 0.41 * ln(rank): with unit-variance logit noise
    the factor 0.41 makes the fitted log-log slope of pairs against rank -1.1). Layer l+1's input is layer l's output scaled to unit RMS
    per token. The router projection and that rescale are torch calls (they sit outside the path);
    route / grouped gate-up / grouped down / combine are this library's kernels."""
    from fngine_b200 import moe, prefill, synth
    layers = [moe.synth_layer(FMT, FMT, INTER, EXPERTS, 5000 + l) for l in range(n_layers)]
    g = torch.Generator(device="cuda").manual_seed(1234)
    routers = [(torch.randn(EXPERTS, HIDDEN, generator=g, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(n_layers)]
    bias = torch.from_numpy(synth.zipf_router_bias(1234)).cuda()
    x0 = torch.randn(tokens, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
    ws = prefill.PrefillWorkspace(tokens, INTER)
    y = torch.empty(tokens, HIDDEN, dtype=torch.float32, device="cuda")

    def step():
        x = x0
        for l in range(n_layers):
            logits = (x @ routers[l].t()).float() + bias
            prefill.moe_layer_prefill(logits, layers[l], x, ws, y)
            x = (y * torch.rsqrt(y.pow(2).mean(dim=1, keepdim=True) + 1e-12)).to(torch.bfloat16)
        return x

    def timed_stack():
        step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            o = step()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / steps, o

    # both hand-offs between the down projection and the combine are timed; the faster one is reported
    prefill.set_accumulation(True)
    ms_fixed, out_fixed = timed_stack()
    prefill.set_accumulation(False)
    ms_pairs, out = timed_stack()
    counts = ws.ints(ws.ws.expert_count, EXPERTS)
    accumulation = {"fixed_point_atomics_ms": ms_fixed, "per_pair_rows_ms": ms_pairs,
                    "reported": "fixed_point_atomics" if ms_fixed < ms_pairs else "per_pair_rows"}
    ms = min(ms_fixed, ms_pairs)
    if ms_fixed < ms_pairs:
        out = out_fixed
        prefill.set_accumulation(True)
    # the two grouped GEMMs of one layer, timed alone
    logits = (x0 @ routers[0].t()).float() + bias
    prefill.moe_route(logits, x0, None, 0, None, None, tokens, ws)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    ev[0].record()
    prefill.moe_grouped_gate_up(layers[0], None, x0, tokens, ws)
    ev[1].record()
    prefill.moe_grouped_down(layers[0], None, tokens, ws)
    ev[2].record()
    torch.cuda.synchronize()
    flops_layer = float(tokens) * TOPK * 7864320.0
    peaks_json = os.path.join(ROOT, "MEASURED_PEAKS.json")
    bf16_peak = float(json.load(open(peaks_json))["bf16_tflops_sustained"]) if os.path.exists(peaks_json) else 1400.0
    tfl = flops_layer * n_layers / (ms * 1e-3) / 1e12
    res = {"workload": "%d layers x %d tokens, 512 IQ3_S experts/layer, top-10, Zipf(1.1) router bias" % (n_layers, tokens),
           "tokens_per_s": tokens / (ms * 1e-3), "ms_per_stack": ms, "tflops": tfl,
           "numerics": "bf16 weights (exact dequant, rounded) x bf16 activations, fp32 accumulate (reference prefill family)",
           "roofline": {"bound": "tensor", "achieved": tfl, "peak": bf16_peak, "unit": "TFLOP/s", "frac": tfl / bf16_peak,
                        "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (of measured)"},
           "gate_up_ms_layer0": ev[0].elapsed_time(ev[1]), "down_ms_layer0": ev[1].elapsed_time(ev[2]),
           "gate_up_tflops_layer0": flops_layer * 2 / 3 / (ev[0].elapsed_time(ev[1]) * 1e-3) / 1e12,
           "down_tflops_layer0": flops_layer / 3 / (ev[1].elapsed_time(ev[2]) * 1e-3) / 1e12,
           "down_to_combine": accumulation,
           "busiest_expert_pairs_last_layer": int(counts.max()), "median_expert_pairs_last_layer": int(np.median(counts)),
           "device_status": ws.status(), "finite_output": bool(torch.isfinite(out.float()).all().item()),
           "timed_region_includes": "torch router projection + unit-RMS rescale between layers"}
    try:  # the CPU path beside it, on a bounded sample (reported, not a target)
        n_cpu = 256
        ids_cpu = ws.ints(ws.ws.topk_expert, tokens * TOPK).reshape(tokens, TOPK)[:n_cpu]
        x_bits = x0[:n_cpu].view(torch.int16).cpu().numpy().view(np.uint16)
        pairs_s, pairs, threads, kind = prefill_cpu_baseline(5000, x_bits, ids_cpu)
        res["cpu_baseline"] = {"value": pairs_s / TOPK, "unit": "tokens/s per layer", "cores": threads, "kind": kind,
                               "sample": "layer 0, first %d tokens with their routing: %d (token, expert) pairs, experts "
                                         "spread over the cores; the GPU figure for one layer is %.0f tokens/s" % (
                                             n_cpu, pairs, tokens * n_layers / (ms * 1e-3))}
    except Exception as exc:  # the oracle is a checker, never a dependency of the measurement
        res["cpu_baseline"] = {"unavailable": type(exc).__name__}
    prefill.set_accumulation(False)
    del layers
    torch.cuda.empty_cache()
    return res


def run_ours(args, rank, world, local_rank):
    import torch
    from fngine_b200 import lib as fblib
    from fngine_b200 import moe, synth
    fblib.load()  # fails loudly when the CUDA library is missing: there is no CPU path
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        return run_ours_multi(args, rank, world, local_rank)

    B, Lr = args.batch, args.layers
    layers, routers, xs_host, xs = [], [], [], []
    for l in range(Lr):
        layers.append(moe.synth_layer(FMT, FMT, INTER, EXPERTS, 5000 + l))
        wr = synth.router_weights(9000 + l)
        routers.append(torch.from_numpy(wr.view(np.int16)).cuda().view(torch.bfloat16))
        xh = torch.from_numpy(synth.activations(7000 + l, B)).pin_memory()
        xs_host.append(xh)
        xs.append(xh.cuda())
    ws = moe.DecodeWorkspace(layers[0])
    y = torch.empty(B, HIDDEN, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    def step():
        for l in range(Lr):
            moe.moe_layer_decode(routers[l], layers[l], xs[l], ws, y)

    # distinct experts per layer (the routing is a function of the seeded inputs only)
    distinct, ids_layer0 = [], None
    for l in range(Lr):
        moe.moe_layer_decode(routers[l], layers[l], xs[l], ws, y)
        torch.cuda.synchronize()
        wk = ws.work()
        distinct.append(wk.n_items)
        if l == 0:
            ids_layer0 = (np.array([list(wk.topk_expert[t]) for t in range(B)], dtype=np.int32),
                          np.array([list(wk.topk_weight[t]) for t in range(B)], dtype=np.float32))
    step_bytes = sum(d * BLOB + ROUTER_BYTES for d in distinct)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)

    # device time of the dominant kernel over the same steps: the expert kernel (gate/up and down tiles of every
    # routed expert in one persistent launch), bracketed by events on the launching stream; then the same two
    # projections as the separate gate/up and down launches of the reference's call sequence
    evs = []
    for _ in range(args.steps):
        for l in range(Lr):
            moe.router_logits(routers[l], xs[l], ws.logits)
            moe.moe_select_publish(ws.logits, xs[l], None, 0, None, None, B, ws)
            a, b = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            a.record()
            moe.moe_hot_experts(layers[l], B, ws)
            b.record()
            moe.moe_combine(ws, None, None, 0, None, None, None, y, B)
            evs.append((l, a, b))
    torch.cuda.synchronize()
    ex_ms = [a.elapsed_time(b) for (_, a, b) in evs]
    ex_bytes = [distinct[l] * BLOB for (l, _a, _b) in evs]
    evs2 = []
    for _ in range(min(args.steps, 4)):
        for l in range(Lr):
            moe.router_logits(routers[l], xs[l], ws.logits)
            moe.moe_select_publish(ws.logits, xs[l], None, 0, None, None, B, ws)
            a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
            moe.moe_hot_gate_up(layers[l], B, ws)
            b.record()
            moe.moe_hot_down(layers[l], B, ws)
            c.record()
            evs2.append((l, a, b, c))
    torch.cuda.synchronize()
    gu_ms = [a.elapsed_time(b) for (_, a, b, _) in evs2]
    dn_ms = [b.elapsed_time(c) for (_, _, b, c) in evs2]
    gu_bytes = [distinct[l] * (BLOB * 2 // 3) for (l, *_r) in evs2]
    dn_bytes = [distinct[l] * (BLOB // 3) for (l, *_r) in evs2]

    # end to end through the host entry point: pinned host x in, host y out, every layer
    yh = torch.empty(B, HIDDEN, dtype=torch.float32).pin_memory()
    xd = torch.empty(B, HIDDEN, dtype=torch.float32, device="cuda")
    for l in range(Lr):
        moe.moe_layer_decode_host(routers[l], layers[l], xs_host[l], ws, xd, y, yh)
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        for l in range(Lr):
            moe.moe_layer_decode_host(routers[l], layers[l], xs_host[l], ws, xd, y, yh)
    f1.record()
    torch.cuda.synchronize()
    e2e_ms = f0.elapsed_time(f1)
    clocks = sampler.stop()
    status = ws.status()

    # other batch sizes of the same layer definition, CUDA-graph replayed (launch-bound otherwise)
    sections = set("batches,cpu,iq4nl,fp8,fp8dec,prefill,legacy".split(",")) if args.sections == "all" else \
        set(x for x in args.sections.split(",") if x and x != "none")

    def want(name):
        return name in sections

    other = {}
    for b2 in ((1, 4) if want("batches") else ()):
        xs2 = [x[:b2].contiguous() for x in xs]
        d2 = []
        for l in range(Lr):
            moe.moe_layer_decode(routers[l], layers[l], xs2[l], ws, y)
            torch.cuda.synchronize()
            d2.append(ws.work().n_items)
        g = torch.cuda.CUDAGraph()
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            with torch.cuda.graph(g, stream=s):
                for l in range(Lr):
                    moe.moe_layer_decode(routers[l], layers[l], xs2[l], ws, y)
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(args.steps):
            g.replay()
        g1.record()
        torch.cuda.synchronize()
        t = g0.elapsed_time(g1) / args.steps
        by = sum(d * BLOB + ROUTER_BYTES for d in d2)
        other[str(b2)] = {"gbs": by / t / 1e6, "us_per_layer": t / Lr * 1e3, "distinct_experts_mean": sum(d2) / Lr,
                          "timing": "CUDA graph of %d layers" % Lr}
    single = single_expert_section(torch, layers, routers, args.steps) if want("batches") else None

    # CPU baseline beside it: the same layer-0 step on the host cores, bounded to ~10 s
    threads = os.cpu_count() or 1
    run_cpu, cpu_bytes, kind = cpu_layer_runner(5000, xs_host[0].numpy(), ids_layer0[0], ids_layer0[1], threads)
    y_cpu = run_cpu()
    t0 = time.perf_counter()
    reps = 0
    cpu_budget_s = (10.0 if kind == "reference" else 1.0) if want("cpu") else 0.0
    while True:
        run_cpu()
        reps += 1
        if time.perf_counter() - t0 > cpu_budget_s or reps >= 2000:
            break
    cpu_dt = (time.perf_counter() - t0) / reps
    # the GPU result of that layer against the CPU result (parity of the measured workload)
    moe.moe_layer_decode(routers[0], layers[0], xs[0], ws, y)
    torch.cuda.synchronize()
    yg = y.cpu().numpy()
    parity = float(max(np.linalg.norm(yg[t] - y_cpu[t]) / np.linalg.norm(y_cpu[t]) for t in range(B)))

    del layers
    torch.cuda.empty_cache()
    iq4 = iq4nl_section(torch, args.steps) if want("iq4nl") else None
    fp8 = fp8_gemm_section(torch) if want("fp8") else None
    fp8dec = fp8_decode_section(torch) if want("fp8dec") else None
    other_formats = None
    if want("iq4nl"):  # the reference pool's own default pair (IQ2_S gate/up, IQ4_NL down, 640) and a Q2_0 down
        other_formats = {"iq2s_iq4nl_640": iq4nl_section(torch, args.steps, fg=22, fd=20, inter=640, batches=(1, 8)),
                         "iq4xs_q2_0_512": iq4nl_section(torch, args.steps, fg=23, fd=42, inter=512, batches=(8,))}
    pre = prefill_section(torch, n_layers=args.prefill_layers) if want("prefill") else None
    try:  # test infrastructure beside the measurement: never allowed to break it
        legacy = legacy_section(torch, steps=args.steps) if want("legacy") else None
    except Exception as exc:
        legacy = {"unavailable": "%s: %s" % (type(exc).__name__, exc)}
    peak, peak_src = peaks()
    ex_ach = sum(ex_bytes) / (sum(ex_ms) * 1e-3) / 1e9
    value = step_bytes * args.steps / (ms * 1e-3) / 1e9
    line = {
        "metric": "iq3s_expert_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8", "data": "synthetic", "config": workload_config(args, Lr),
        "tokens_per_s": B * Lr * args.steps / (ms * 1e-3),
        "us_per_layer": ms / args.steps / Lr * 1e3,
        "distinct_experts_per_layer": distinct,
        "frac_of_hbm_peak": value / peak,
        "roofline": {"bound": "hbm", "kernel": "experts_kernel<IQ3_S> (selection, then gate/up + down tiles of every routed expert, one launch)",
                     "achieved": ex_ach, "peak": peak, "unit": "GB/s", "frac": ex_ach / peak, "peak_source": peak_src,
                     "traffic": EXPERTS_DRAM_TRAFFIC_RATIO * sum(ex_bytes) / len(ex_bytes),
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on layer 0 of this "
                                       "workload (239.30 MB for 234.85 MB algorithmic), scaled by the expert count of "
                                       "each layer",
                     "us_per_launch": sum(ex_ms) / len(ex_ms) * 1e3,
                     "algorithmic_bytes_per_launch": sum(ex_bytes) / len(ex_bytes),
                     "algorithmic_bytes": "distinct routed experts x 1,689,600 B (gate + up + down of an IQ3_S expert)",
                     "as_separate_launches": {
                         "gate_up": {"achieved": sum(gu_bytes) / (sum(gu_ms) * 1e-3) / 1e9,
                                     "us_per_launch": sum(gu_ms) / len(gu_ms) * 1e3},
                         "down": {"achieved": sum(dn_bytes) / (sum(dn_ms) * 1e-3) / 1e9,
                                  "us_per_launch": sum(dn_ms) / len(dn_ms) * 1e3}}},
        "cpu_baseline": {"value": cpu_bytes / cpu_dt / 1e9, "unit": "GB/s", "cores": threads, "kind": kind,
                         "sample": "layer 0 of the same workload (batch %d, %d distinct experts), %d repetitions, "
                                   "%.2f ms each" % (B, distinct[0], reps, cpu_dt * 1e3)},
        "e2e": {"value": step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": B * HIDDEN * 4 * Lr, "d2h_bytes_per_step": B * HIDDEN * 4 * Lr,
                "ms_per_step": e2e_ms / args.steps,
                "api": "fb_moe_layer_decode_host per layer: pinned host x in, host y out, stream wait inside"},
        "gpu_launches": args.steps * Lr * 3,
        "other_batches": other,
        "single_expert": single,
        "iq4nl_decode": iq4,
        "other_formats_decode": other_formats,
        "fp8_row_gemm": fp8,
        "fp8_row_decode": fp8dec,
        "prefill_stack": pre,
        "reference_gpu_kernels_same_box": legacy,
        "parity_vs_cpu_max_rel_l2": parity,
        "device_status": status,
        "clocks": clocks,
    }
    print(json.dumps(line))


def ep_prefill_section(rank, world, n_layers=48, tokens=8192, steps=2, parity_tokens=2, spare_slots=4):
    """The 48-layer prefill stack of bench.py's single-GPU section, expert-parallel: same seeds, same
    router bias, tokens data-parallel. Two placements of the experts are timed one after the other:
    contiguous shards (expert e on rank e // (512 / N)), which also serve as the profiling pass that records
    every layer's routing histogram, and the placement planned from that profile (fngine_b200/placement.py:
    experts spread by load, the hottest copied into `spare_slots` extra slots per rank). The headline
    tokens_per_s is the planned placement's. Returns the section dict on rank 0 (None on the other ranks).
    Timed on the device, barrier on both sides, max over ranks."""
    import torch
    import torch.distributed as dist
    from fngine_b200 import placement, prefill, synth
    from fngine_b200.ep_prefill import (EpPrefillScratch, EpPrefillShard, comm_pointer, ep_prefill_layer,
                                        ep_prefill_layer_c, topk)
    FMT, INTER = 21, 512
    g = torch.Generator(device="cuda").manual_seed(1234)
    routers = [(torch.randn(EXPERTS, HIDDEN, generator=g, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(n_layers)]
    bias = torch.from_numpy(synth.zipf_router_bias(1234)).cuda()
    x0 = torch.randn(tokens, HIDDEN, generator=g, device="cuda").to(torch.bfloat16)
    tl = tokens // world
    x_local = x0[rank * tl:(rank + 1) * tl].contiguous()
    ws = prefill.PrefillWorkspace(tokens, INTER)  # a rank may receive a row of every token
    totals = {"rows_received": 0, "dispatch_bytes": 0, "combine_bytes": 0}
    hist = torch.zeros(n_layers, EXPERTS, dtype=torch.int64, device="cuda")
    shards = []
    combine = "all_to_all"
    c_call = None  # (communicator, scratch, y buffer): the layer through fb_ep_prefill_layer instead of the mirror

    def step(record=False):
        x = x_local
        for l in range(n_layers):
            logits = (x @ routers[l].t()).float() + bias
            if record:
                hist[l] += torch.bincount(topk(logits)[0].reshape(-1).long(), minlength=EXPERTS)
            if c_call is not None:
                y, st = ep_prefill_layer_c(logits, x, shards[l], ws, c_call[1], c_call[2], c_call[0]), None
            else:
                y, st = ep_prefill_layer(logits, x, shards[l], ws, combine=combine)
            if record:
                for k in totals:
                    totals[k] += st[k]
            x = (y * torch.rsqrt(y.pow(2).mean(dim=1, keepdim=True) + 1e-12)).to(torch.bfloat16)
        return x

    def timed():
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            out_ = step()
        b.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([a.elapsed_time(b) / steps], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), out_

    # 1. contiguous shards: the profiling pass (routing histograms of every layer) and the first timing
    shards = [EpPrefillShard(rank, world, 5000 + l, FMT, INTER) for l in range(n_layers)]
    step(record=True)
    dist.all_reduce(hist)
    step()
    ms_contiguous, _ = timed()
    load = hist.cpu().numpy().astype(np.float64)
    contiguous = placement.Placement.contiguous(world)
    plans = [placement.plan_placement(load[l], world, EXPERTS // world + spare_slots) for l in range(n_layers)]
    balance = {"contiguous_shards": float(np.mean([contiguous.imbalance(load[l]) for l in range(n_layers)])),
               "planned": float(np.mean([plans[l].imbalance(load[l]) for l in range(n_layers)])),
               "planned_worst_layer": float(max(plans[l].imbalance(load[l]) for l in range(n_layers))),
               "experts_copied_per_layer": float(np.mean([sum(len(c) > 1 for c in p.copies) for p in plans])),
               "spare_slots_per_rank": spare_slots,
               "what": "pairs on the busiest rank / mean over the ranks, averaged over the layers, from the routing "
                       "histogram of the profiling pass (the timed passes route the same way)"}
    # 2. the planned placement: what the section reports
    del shards
    torch.cuda.empty_cache()
    shards = [EpPrefillShard(rank, world, 5000 + l, FMT, INTER, placement=plans[l]) for l in range(n_layers)]

    # layer 0 alone, for the parity check of the measured workload
    logits0 = (x_local @ routers[0].t()).float() + bias
    y_l0, _ = ep_prefill_layer(logits0, x_local, shards[0], ws)
    e0_, w0_ = topk(logits0)
    step()
    ms_a2a, out = timed()
    # 3. the same placement with the combine as one reduce-scatter instead of all-to-all + owner sum
    combine = "reduce_scatter"
    step()
    ms_rs, out_rs = timed()
    # (the two are compared on one layer: the stack is a random deep network without residuals, in which a
    # last-bit difference flips a near-tie of some token's top-10 a few layers on and the outputs part)
    y_l0_rs, _ = ep_prefill_layer(logits0, x_local, shards[0], ws, combine="reduce_scatter")
    rs_vs_a2a = float(((y_l0_rs - y_l0).norm() / y_l0.norm()).item())
    if ms_rs <= ms_a2a:
        ms, out = ms_rs, out_rs
    else:
        ms = ms_a2a
    # 4. the same layers through the one C entry point (fb_ep_prefill_layer) on torch's communicator
    comm = comm_pointer()
    y_c = torch.empty(tl, HIDDEN, dtype=torch.float32, device="cuda")
    ms_c, c_equal = {}, None
    for comb in ("all_to_all", "reduce_scatter"):
        c_call = (comm, EpPrefillScratch(tl, world, comb), y_c)
        if comb == "all_to_all":
            c_equal = bool(torch.equal(ep_prefill_layer_c(logits0, x_local, shards[0], ws, c_call[1], y_c, comm), y_l0))
        step()
        ms_c[comb], out_c = timed()
        if ms_c[comb] < ms:
            ms, out = ms_c[comb], out_c
    c_call = None
    eq = torch.tensor([float(c_equal)], device="cuda")
    dist.all_reduce(eq, op=dist.ReduceOp.MIN)
    c_equal = bool(eq.item())
    agg = torch.tensor([float(totals[k]) for k in ("rows_received", "dispatch_bytes", "combine_bytes")], device="cuda")
    mx = agg.clone()
    dist.all_reduce(agg)
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    finite = torch.tensor([float(torch.isfinite(out.float()).all().item()), float(ws.status() == 0)], device="cuda")
    dist.all_reduce(finite, op=dist.ReduceOp.MIN)
    if rank != 0:
        return None
    parity = None
    try:
        from oracle import oracle as O
        ids, w = e0_[:parity_tokens].cpu().numpy(), w0_[:parity_tokens].cpu().numpy()
        xb = x_local[:parity_tokens].view(torch.int16).cpu().numpy().view(np.uint16)
        got = y_l0[:parity_tokens].cpu().numpy()
        errs = []
        for t_ in range(parity_tokens):
            want = np.zeros(HIDDEN, dtype=np.float32)
            for e, wt in sorted(zip(ids[t_].tolist(), w[t_].tolist())):
                _, ye = O.expert_ffn_bf16(FMT, FMT, HIDDEN, INTER, synth.expert_blob(FMT, FMT, INTER, 5000, int(e)), xb[t_:t_ + 1])
                want += np.float32(wt) * ye[0]
            errs.append(float(np.linalg.norm(got[t_] - want) / np.linalg.norm(want)))
        parity = max(errs)
    except Exception as exc:  # the oracle is a checker, never a dependency of the measurement
        parity = "oracle unavailable: %s" % type(exc).__name__
    flops = float(tokens) * TOPK * 7864320.0 * n_layers
    peaks_json = os.path.join(ROOT, "MEASURED_PEAKS.json")
    bf16_peak = float(json.load(open(peaks_json))["bf16_tflops_sustained"]) if os.path.exists(peaks_json) else 1400.0
    tfl = flops / (ms * 1e-3) / 1e12
    return {"workload": "%d layers x %d tokens, 512 IQ3_S experts/layer, top-10, Zipf(1.1) router bias; ep%d: %d experts "
                        "per GPU, %d tokens per GPU" % (n_layers, tokens, world, EXPERTS // world, tl),
            "tokens_per_s": tokens / (ms * 1e-3), "ms_per_stack": ms, "tflops": tfl, "scaling": "strong",
            "placement": "planned from the routing profile of a first pass: experts spread over the ranks by load, "
                         "the hottest copied (their pairs split by row number)",
            "pair_load_max_over_mean": balance,
            "contiguous_shards": {"ms_per_stack": ms_contiguous, "tokens_per_s": tokens / (ms_contiguous * 1e-3)},
            "combine": {"all_to_all_plus_owner_sum_ms": ms_a2a, "reduce_scatter_ms": ms_rs,
                        "reported": "reduce_scatter" if ms_rs <= ms_a2a else "all_to_all",
                        "layer0_rel_l2_between_the_two": rs_vs_a2a},
            "c_entry_point": {"what": "the same stack with every layer enqueued by one fb_ep_prefill_layer call on the "
                                      "process group's ncclComm_t (all collectives on the compute stream)",
                              "all_to_all_plus_owner_sum_ms": ms_c["all_to_all"], "reduce_scatter_ms": ms_c["reduce_scatter"],
                              "layer0_bit_equal_to_the_python_mirror": c_equal},
            "roofline": {"bound": "tensor", "achieved": tfl / world, "peak": bf16_peak, "unit": "TFLOP/s per GPU",
                         "frac": tfl / world / bf16_peak,
                         "peak_source": "MEASURED_PEAKS.json bf16_tflops_sustained (of measured)"},
            "rows_received_per_stack": {"sum": agg[0].item(), "max_rank": mx[0].item()},
            "all_to_all_bytes_per_stack": {"dispatch": agg[1].item(), "combine": agg[2].item(),
                                           "max_rank_dispatch": mx[1].item(), "max_rank_combine": mx[2].item()},
            "collectives_per_layer": "dense exchange: all-gather of bf16 rows + all-gather of (expert, weight) lists + one "
                                     "fixed-size fp32 all-to-all, rank-order sum on the owner (NCCL; no host sync)",
            "parity_layer0_max_rel_l2": parity, "parity_tokens": parity_tokens,
            "finite_output": bool(finite[0].item()), "device_status_ok": bool(finite[1].item()),
            "timed_region_includes": "torch router projection + unit-RMS rescale between layers, dispatch gather"}


def run_ours_multi(args, rank, world, local_rank):
    """bench.py for N > 1: strong scaling of the same 16-token decode step over expert-parallel ranks.
    The timed step exchanges through peer memory inside the kernels (fb_moe_layer_decode_ep_p2p); the
    same step with NCCL all-to-alls is timed beside it and the two results are compared bit for bit."""
    import torch
    import torch.distributed as dist
    from fngine_b200 import ep, moe, synth
    from fngine_b200.ep import EpDecodeLayer, PeerExchange, ep_layer_step, layer_decode_ep_p2p, token_range

    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B, Lr = args.batch, args.layers
    lo, hi = token_range(rank, world, B)
    layers, routers, xs_host, xs = [], [], [], []
    for l in range(Lr):
        layers.append(EpDecodeLayer(rank, world, 5000 + l))
        wr = synth.router_weights(9000 + l)
        routers.append(torch.from_numpy(wr.view(np.int16)).cuda().view(torch.bfloat16))
        xh = torch.from_numpy(synth.activations(7000 + l, B)[lo:hi].copy()).pin_memory()
        xs_host.append(xh)
        xs.append(xh.cuda())
    ws = moe.DecodeWorkspace(layers[0].layer)
    bufs = {"y_partial": torch.empty(B, HIDDEN, dtype=torch.float32, device="cuda"),
            "y_local": torch.empty(hi - lo, HIDDEN, dtype=torch.float32, device="cuda")}
    xchg = PeerExchange(rank, world)
    y_p2p = torch.empty(hi - lo, HIDDEN, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()

    def step_nccl():
        for l in range(Lr):
            ep_layer_step(routers[l], layers[l], xs[l], ws, bufs)

    def step():
        for l in range(Lr):
            layer_decode_ep_p2p(routers[l], layers[l], xs[l], ws, xchg, y_p2p)

    # the two exchanges give the same bits (same partial rows, same rank-order sum)
    same = True
    for l in range(Lr):
        y_a = ep_layer_step(routers[l], layers[l], xs[l], ws, bufs).clone()
        layer_decode_ep_p2p(routers[l], layers[l], xs[l], ws, xchg, y_p2p)
        torch.cuda.synchronize()
        same = same and bool(torch.equal(y_a, y_p2p))
    flag = torch.tensor([1.0 if same else 0.0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    same = bool(flag.item() == 1.0)

    # local distinct experts per layer (for the byte count) and a parity check of layer 0 on rank 0
    distinct = []
    for l in range(Lr):
        ep_layer_step(routers[l], layers[l], xs[l], ws, bufs)
        torch.cuda.synchronize()
        distinct.append(ws.work().n_items)
        if l == 0:
            layer_decode_ep_p2p(routers[l], layers[l], xs[l], ws, xchg, y_p2p)
            torch.cuda.synchronize()
            y0 = y_p2p.clone()
    local_bytes = torch.tensor([float(sum(d * BLOB + ROUTER_BYTES for d in distinct))], device="cuda")
    dist.all_reduce(local_bytes)
    step_bytes = float(local_bytes.item())

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    # the NCCL all-to-all step beside it
    for _ in range(3):
        step_nccl()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    n0, n1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n0.record()
    for _ in range(args.steps):
        step_nccl()
    n1.record()
    torch.cuda.synchronize()
    dist.barrier()
    tn = torch.tensor([n0.elapsed_time(n1)], device="cuda")
    dist.all_reduce(tn, op=dist.ReduceOp.MAX)
    nccl_ms = float(tn.item())

    # end to end: pinned host rows of the own tokens in, own y rows out, every layer
    yh = torch.empty(hi - lo, HIDDEN, dtype=torch.float32).pin_memory()
    xd = torch.empty(hi - lo, HIDDEN, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    dist.barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.steps):
        for l in range(Lr):
            xd.copy_(xs_host[l], non_blocking=True)
            y = layer_decode_ep_p2p(routers[l], layers[l], xd, ws, xchg, y_p2p)
            yh.copy_(y, non_blocking=True)
            torch.cuda.current_stream().synchronize()
    f1.record()
    torch.cuda.synchronize()
    t2 = torch.tensor([f0.elapsed_time(f1)], device="cuda")
    dist.all_reduce(t2, op=dist.ReduceOp.MAX)
    e2e_ms = float(t2.item())

    clocks = sampler.stop() if rank == 0 else None
    status = ws.status()

    # parity of the measured workload: layer 0 of this rank's tokens against the CPU oracle
    parity = None
    if rank == 0:
        from oracle import oracle as O
        x_full = synth.activations(7000, B)
        wr_bits = synth.router_weights(9000)
        logits = x_full.astype(np.float32) @ synth.bf16_bits_to_f32(wr_bits).T
        ids, w = O.topk(np.ascontiguousarray(logits[:, :EXPERTS]))
        ids, w, xo = ids[lo:hi], w[lo:hi], x_full[lo:hi]
        used = sorted(set(ids.reshape(-1).tolist()))
        blobs = np.concatenate([synth.expert_blob(21, 21, 512, 5000, e) for e in used])
        ids2 = np.vectorize({e: i for i, e in enumerate(used)}.get)(ids).astype(np.int32)
        want = O.moe_layer(21, 21, HIDDEN, 512, blobs, BLOB, xo, ids2, w, threads=os.cpu_count() or 1, lib=O.ref())
        got = y0.cpu().numpy()
        parity = float(max(np.linalg.norm(got[i] - want[i]) / np.linalg.norm(want[i]) for i in range(hi - lo)))
    dist.barrier()
    # the 48-layer prefill stack, expert-parallel (the decode layers are released first)
    pre = None
    if args.sections == "all" or "prefill" in args.sections.split(","):
        del layers
        torch.cuda.empty_cache()
        pre = ep_prefill_section(rank, world, n_layers=args.prefill_layers)
    if rank == 0:
        peak, peak_src = peaks()
        value = step_bytes * args.steps / (ms * 1e-3) / 1e9
        ach = value / world  # per GPU, whole layer step (kernels are timed one by one only at N = 1)
        cfg = workload_config(args, Lr)
        cfg["parallelism"] = ("ep%d: %d experts per GPU, tokens data-parallel (%d per GPU), dispatch + combine by peer "
                              "stores over NVLink inside the kernels (no collective call in the step)" % (
                                  world, EXPERTS // world, B // world))
        line = {"metric": "iq3s_expert_gemv_hbm_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": cfg, "tokens_per_s": B * Lr * args.steps / (ms * 1e-3), "us_per_layer": ms / args.steps / Lr * 1e3,
                "distinct_local_experts_rank0": distinct,
                "nccl_all_to_all_step": {"us_per_layer": nccl_ms / args.steps / Lr * 1e3,
                                         "value": step_bytes * args.steps / (nccl_ms * 1e-3) / 1e9,
                                         "bitwise_equal_to_peer_exchange": same},
                "roofline": {"bound": "hbm", "kernel": "whole expert-parallel layer step, per GPU (incl. the exchange)", "achieved": ach, "peak": peak,
                             "unit": "GB/s", "frac": ach / peak, "peak_source": peak_src, "traffic": None},
                "e2e": {"value": step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                        "h2d_bytes_per_step": (hi - lo) * HIDDEN * 4 * Lr * world,
                        "d2h_bytes_per_step": (hi - lo) * HIDDEN * 4 * Lr * world, "ms_per_step": e2e_ms / args.steps},
                "gpu_launches": args.steps * Lr * 4 * world, "parity_vs_cpu_max_rel_l2": parity,
                "device_status": status, "clocks": clocks, "prefill_stack": pre,
                "cpu_baseline": None}
        print(json.dumps(line))
    xchg.close()
    dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--layers", type=int, default=64,
                    help="MoE layers per step, each with its own 865 MB expert set (48 = the model's depth)")
    ap.add_argument("--prefill-layers", type=int, default=48,
                    help="layers of the prefill stack section (a profiler run wants 1)")
    ap.add_argument("--sections", default="all",
                    help="extra sections beside the headline decode measurement: all | none | comma list of "
                         "batches,cpu,iq4nl,fp8,fp8dec,prefill,legacy (a profiler run wants none)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
