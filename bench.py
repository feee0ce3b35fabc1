"""bench.py -- NNCP Transformer-XL train step on 1..8 B200: compressed symbols/s.

  python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
  python bench.py --impl reference ...                     (CPU arm: the oracle port, host cores)

A step is one segment of every stream: forward over [memory | segment], loss, backward,
RMSProp update, memory shift (fwd+bwd+RMSProp, the metric of BASELINE.json).  The workload is
BASELINE config[2] (vocab 16384, 12 layers, d_model 512, 8 heads x 64, d_ff 2048, seg 64,
mem 64, 32 streams, bf16 with fp32 master weights) on seeded synthetic Zipf+Markov token ids;
streams are sharded across ranks and gradients are summed by NCCL all-reduces inside the backward pass.

`value`   device-resident ids/targets, nothing read back (CUDA events, max over ranks).
`e2e`     the same steps through the host-buffer plugin calls: ids from pinned host memory
          every step, the coder-ready prob0 paths and the loss read back every step (encoder order:
          the next segment's forward pass is queued before the host waits for this segment's results).
`roofline` the tcgen05 GEMM kernel: sum of 2*M*N*K over its launches / sum of their CUDA-event
          durations, against the measured bf16 peak.
`attention` the isolated attention op of BASELINE config[1] (forward, and forward + backward)
          through nncu_attention_forward / _backward: TFLOP/s and the fraction of its
          min(tensor, HBM) roofline.
`cpu_baseline` the CPU oracle (port of nncp.c's graph, OpenMP) timed on a bounded sample.

  python bench.py --mode words     the word tokenizer (host code, no GPU) beside the reference's tool

The K-step timed region is measured REPEATS times in the same process (each bracketed by a
barrier and a synchronize, CUDA events, max over ranks); `value` is the median, `value_min` /
`value_max` the spread.
"""
import argparse
import ctypes as C
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

CONFIGS = {
    # BASELINE.json configs[2]
    "c2": dict(n_layer=12, d_model=512, n_head=8, d_key=64, d_inner=2048, d_pos=128, mem_len=64,
               seg_len=64, n_streams=32, n_symbols=16384, use_bf16=1),
    # BASELINE.json configs[0]
    "c0": dict(n_layer=2, d_model=128, n_head=4, d_key=32, d_inner=512, d_pos=64, mem_len=32,
               seg_len=32, n_streams=4, n_symbols=256, use_bf16=0),
    # BASELINE.json configs[3] (64 streams over all ranks) and the train step of configs[4]
    "c3": dict(n_layer=20, d_model=1024, n_head=16, d_key=64, d_inner=4096, d_pos=320, mem_len=256,
               seg_len=64, n_streams=64, n_symbols=16384, use_bf16=1),
    "c4": dict(n_layer=12, d_model=512, n_head=8, d_key=64, d_inner=2048, d_pos=576, mem_len=512,
               seg_len=64, n_streams=128, n_symbols=16384, use_bf16=1),
}
# streams of the bounded CPU sample (the CPU port needs about half a second per c2 stream-step)
CPU_STREAMS = {"c2": 2, "c3": 1, "c4": 2}
COMMON = dict(use_bias=1, use_w_r=1, tied_w_r=0, tied_b_r=0, query_bias=1, ln_flags=1, ff_act=1,
              init_range=0.02, init_kind=1, seed=123, lr=3e-4, beta2=0.99, eps=1e-8)


def step_flops(c, B):
    """Algorithmic FLOPs of one train step (2*m*n*k per contraction; bwd = dX + dW, no dX into
    the memory rows)."""
    D, H, dk, F, T, M, V, P = (c["d_model"], c["n_head"], c["d_key"], c["d_inner"], c["seg_len"],
                               c["mem_len"], c["n_symbols"], c["d_pos"])
    L, HD = M + T, c["n_head"] * c["d_key"]
    F1 = 2 * F if c.get("ff_act", 1) in (2, 3) else F
    layer = (2 * B * T * D * HD + 2 * B * L * D * 2 * HD + 2 * B * H * T * L * dk + 2 * B * H * T * P * dk +
             2 * B * H * T * L * dk + 2 * B * T * HD * D + 2 * B * T * D * F1 + 2 * B * T * F * D)
    head = 2 * B * T * D * V
    fwd = c["n_layer"] * layer + head
    return 3 * fwd - c["n_layer"] * 2 * B * M * D * 2 * HD


def synth_tokens(n, V, seed=1234, lam=0.5):
    """Zipf(s=1.1) unigram mixed (lambda 0.5) with an order-1 Markov chain whose rows put
    Dirichlet(0.05) mass on 512 successors drawn from the most frequent ranks."""
    rng = np.random.default_rng(seed)
    ranks = np.arange(1, V + 1, dtype=np.float64)
    uni = ranks ** -1.1
    uni /= uni.sum()
    n_ctx = min(V, 4096)  # contexts beyond this rank share rows (bounded generator memory)
    succ = rng.integers(0, 512, size=(n_ctx, 16))
    w = rng.dirichlet(np.full(16, 0.05 * 32), size=n_ctx)
    cw = np.cumsum(w, axis=1)
    out = np.empty(n, np.int32)
    u_draw = rng.choice(V, size=n, p=uni)
    pick = rng.random(n)
    mix = rng.random(n) < lam
    prev = 0
    for i in range(n):
        if mix[i]:
            prev = u_draw[i]
        else:
            r = prev % n_ctx
            prev = succ[r, min(int(np.searchsorted(cw[r], pick[i])), 15)]
        out[i] = prev
    return out


def make_batches(c, B_total, steps, seed=1234):
    """ids/targets [steps][T][B_total] laid out as process_block does (nncp.c:2945-3001): stream b
    owns a contiguous slice; the input at position t is the symbol at t-1 (0 at a stream start)."""
    T, V = c["seg_len"], c["n_symbols"]
    per_stream = steps * T
    if V <= 256:
        rng = np.random.default_rng(seed)
        toks = rng.integers(0, V, B_total * per_stream).astype(np.int32)
    else:
        toks = synth_tokens(B_total * per_stream, V, seed)
    s = toks.reshape(B_total, per_stream)
    prev = np.concatenate([np.zeros((B_total, 1), np.int32), s[:, :-1]], 1)
    ids = prev.reshape(B_total, steps, T).transpose(1, 2, 0)
    tg = s.reshape(B_total, steps, T).transpose(1, 2, 0)
    return np.ascontiguousarray(ids), np.ascontiguousarray(tg)


class ClockSampler:
    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names)
                   if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return (p.get("bf16_tflops_sustained", 1420.5), p.get("hbm_gbs", 6453.4), "measured",
                p.get("bf16_tflops", 1693.0))
    return 1400.0, 6650.0, "fallback", 1590.0


def cpu_port_run(c, steps, warmup, streams):
    """Times the CPU oracle on `streams` streams of the workload's model; returns symbols/s."""
    pkg = entry._package()
    from oracle import oracle as orc
    # every host core, whatever OMP_NUM_THREADS the launcher exported (torch.distributed.run sets 1)
    threads = orc.lib().orc_set_threads(os.cpu_count() or 1)
    kw = dict(COMMON)
    kw.update(c)
    kw.update(n_streams=streams, n_streams_total=streams, use_bf16=0)
    p = pkg.abi.make_params(**kw)
    m = orc.OracleModel(p)
    ids, tg = make_batches(c, streams, steps + warmup, seed=99)
    m.reset()
    t0 = None
    for s in range(steps + warmup):
        if s == warmup:
            t0 = time.perf_counter()
        m.L.orc_eval(m.h, -1, ids[s].ctypes.data_as(C.c_void_p), None)
        m.eval_gradient(tg[s])
        m.update()
    dt = time.perf_counter() - t0
    m.close()
    return steps * c["seg_len"] * streams / dt, dt, threads


def workload_name(name, c):
    return (f"{name}: NNCP Transformer-XL train step, vocab {c['n_symbols']}, {c['n_layer']} layers, "
            f"d_model {c['d_model']}, {c['n_head']}x{c['d_key']} heads, d_ff {c['d_inner']}, "
            f"seg {c['seg_len']}, mem {c['mem_len']}, {c['n_streams']} streams")


def job_config(name, c, world, exchange):
    """The `config` object of the JSON line; both arms print the same one for the same N."""
    return {"workload": workload_name(name, c), "streams_per_gpu": c["n_streams"] // world,
            "parallelism": f"dp{world} over streams", "gradient_exchange": exchange,
            "l2": "per-step working set (weights, optimizer state, activations) exceeds the 126 MB L2",
            "tokens": "seeded Zipf(1.1)+order-1 Markov ids (stand-in for tokenised text)"}


def exchange_name(world):
    if world == 1:
        return "none"
    if os.environ.get("NNCU_PY_ALLREDUCE") == "1":
        return "one all-reduce after backward"
    if os.environ.get("NNCU_SHARDED_UPDATE") == "1":
        return ("per-layer reduce-scatter, RMSProp on the rank's shard, all-gather of the bf16 weights; small parameters "
                "all-reduced; embedding gradient from gathered ids and rows (Ring / LL128 / 32 channels pinned)")
    per = os.environ.get("NNCU_BUCKET_LAYERS") or ("2" if world >= 8 else "1")
    return (f"NCCL all-reduce of {per} layer(s) at a time inside the backward pass (overlapped; Ring / LL128 / 32 channels "
            "pinned), every rank applies the whole RMSProp step; embedding gradient from gathered ids and rows instead of "
            "the dense table")


def shipped_cpu_codec():
    """The reference's own `--cpu` code path as it ships (nncp_original_compress / _decompress): a
    range coder behind a uniform 1/256 model, no network, one thread.  Timed on 1 MiB of seeded bytes
    below 200 (its decoder stops at the first decoded 0xFF).  Not the path this repository builds: a
    side record, so that what the reference can run on a CPU stands beside the figures."""
    from oracle import oracle as orc
    L = orc.cpu_codec_ref()
    if L is None:
        return None
    n = 1 << 20
    src = np.random.default_rng(1234).integers(0, 200, n, dtype=np.uint8)
    out, back = np.zeros(2 * n + 1024, np.uint8), np.zeros(n + 16, np.uint8)
    n_out, n_back = C.c_size_t(), C.c_size_t()
    # the codec reports on the C library's stdout: that goes to /dev/null so that this process still
    # prints one JSON line (flushed before the descriptor comes back, or it would surface at exit)
    libc = C.CDLL(None)
    sys.stdout.flush()
    saved, null = os.dup(1), os.open(os.devnull, os.O_WRONLY)
    os.dup2(null, 1)
    try:
        t0 = time.perf_counter()
        ok = L.nncp_original_compress(src.ctypes.data, n, out.ctypes.data, out.size, C.byref(n_out), False)
        t1 = time.perf_counter()
        ok2 = L.nncp_original_decompress(out.ctypes.data, n_out.value, back.ctypes.data, back.size, C.byref(n_back),
                                         False)
        t2 = time.perf_counter()
    finally:
        libc.fflush(None)
        os.dup2(saved, 1)
        os.close(saved)
        os.close(null)
    return {"compress_MB_per_s": n / (t1 - t0) / 1e6, "decompress_MB_per_s": n / (t2 - t1) / 1e6,
            "ratio": n_out.value / n, "round_trip_exact": bool(ok and ok2 and n_back.value == n and
                                                                 np.array_equal(back[:n], src)),
            "cores": 1, "note": "src/metal/nncp_original_port.c compiled unchanged; its model is a uniform "
                                "distribution (no network), so the output is as large as the input"}


def run_reference(args, c):
    """The reference arm: the CPU oracle port of the train step on all host cores (the reference's
    own train step runs on LibNC, which its tree does not contain).  Rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    streams = CPU_STREAMS.get(args.config, c["n_streams"])
    K, W = min(args.steps, 100), min(args.warmup, 5)   # bounded: a c2 step of 2 streams is ~0.4 s of CPU work
    val, dt, threads = cpu_port_run(c, K, W, streams)
    sample = (f"{K} steps of {streams} of the {c['n_streams']} streams x {c['seg_len']} symbols, "
              f"oracle/trf_oracle.c with OpenMP on {threads} threads; the reference's own train step "
              f"needs LibNC, which its tree does not contain")
    line = {"impl": "reference", "metric": "compressed symbols/s (fwd+bwd+RMSProp)", "value": val,
            "unit": "symbols/s", "n_gpus": args.gpus, "steps": K, "warmup": W,
            "ms_per_step": 1e3 * dt / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": job_config(args.config, c, args.gpus, exchange_name(args.gpus)),
            "cpu_baseline": {"value": val, "unit": "symbols/s", "cores": threads, "kind": "port",
                             "sample": sample},
            "e2e": {"value": val, "unit": "symbols/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "shipped_cpu_codec": shipped_cpu_codec()}
    print(json.dumps(line), flush=True)


def decode_step_bytes(c, n_floats):
    """Algorithmic HBM bytes of one decode step of all streams: every bf16 weight once except the
    input-embedding table (B rows of it), K and V of the memory and of the segment so far (average
    T/2 rows), the probability tables written once and read once, the prob0 trees written and read."""
    D, T, M, V, B, nl = c["d_model"], c["seg_len"], c["mem_len"], c["n_symbols"], c["n_streams"], c["n_layer"]
    HD = c["n_head"] * c["d_key"]
    weights = 2 * (n_floats - V * D) + 2 * B * D
    kv = nl * B * (M + T // 2) * 2 * HD * 2
    tables = 2 * B * V * 4 + 2 * B * V * 2
    return weights + kv + tables


def run_decode(args, c, name):
    """Decoding: one-symbol steps (forward, prob0 trees and the range decoder on the device, each
    step a CUDA graph), then the train step on the decoded segment.  The stream decoded is the one
    the encoder of the same library produced from seeded synthetic ids; the symbols must come back
    exactly.  One GPU: a single bit stream decodes serially."""
    import torch
    if int(os.environ.get("WORLD_SIZE", "1")) != 1 or args.gpus != 1:
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"mode": "decode", "unavailable": "one coded stream decodes on one GPU"}), flush=True)
        return
    torch.cuda.set_device(0)
    pkg = entry._package()
    lib = pkg.library()
    host = pkg.host
    kw = dict(COMMON)
    kw.update(c)
    kw.update(n_streams_total=c["n_streams"], gemm_backend=args.backend, device=0)
    p = pkg.abi.make_params(**kw)
    T, B, V = c["seg_len"], c["n_streams"], c["n_symbols"]
    K, W = args.steps, max(args.warmup, 3)
    n_seg = W + K
    n = n_seg * T * B
    toks = (synth_tokens(n, V, 4321) if V > 256 else np.random.default_rng(1).integers(0, V, n)).astype(np.uint16)
    fp = host.file_params(p, block_len=n)
    ops = host.bind_cuda(p)      # first use of every kernel in this process: not part of the encode figure
    host.compress(ops, host.file_params(p, block_len=2 * T * B), toks[: 2 * T * B], host.EVAL_SEGMENT, host.OUT_CODER_READY)
    host.unbind_cuda(ops)
    ops = host.bind_cuda(p)
    t0 = time.perf_counter()
    data, st = host.compress(ops, fp, toks, host.EVAL_SEGMENT, host.OUT_CODER_READY)
    t_enc = time.perf_counter() - t0
    host.unbind_cuda(ops)
    _, nsym, used = host.read_header(data)
    payload = data[used:]

    # (1) the segment loop on the model's entry points, K segments timed after W
    m = pkg.TrfModel(p)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    m.set_stream(stream.cuda_stream)
    stride = n // B
    lay = toks.reshape(B, stride)            # stream b owns a contiguous slice (block_len % B == 0 here)
    sampler = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m.reset()
    m.decoder_begin(payload)
    m.set_lr(p.lr)
    ids0 = np.zeros(B, np.int32)
    out = np.zeros((n_seg, T, B), np.int32)
    lib.nncu_profile_begin(0)
    for sgm in range(n_seg):
        if sgm == W:
            torch.cuda.synchronize()
            lib.nncu_profile_begin(0)
            sampler.start()
            tw = time.perf_counter()
            e0.record(stream)
        out[sgm] = m.decode_steps(0, T, ids0)
        m.eval_gradient(out[sgm])
        m.update()
        ids0 = out[sgm, T - 1]
    e1.record(stream)
    torch.cuda.synchronize()
    wall = time.perf_counter() - tw
    clocks = sampler.stop()
    prof = pkg.abi.Profile()
    lib.nncu_profile_end(C.byref(prof))
    consumed = m.decoder_end()
    ms = max(e0.elapsed_time(e1), wall * 1e3)
    exact = bool(np.array_equal(out.transpose(2, 0, 1).reshape(B, stride), lay))
    value = K * T * B / (ms * 1e-3)

    # (2) the decode steps alone (no train step): what the HBM figure is quoted on
    m.reset()
    m.decoder_begin(payload)
    m.decode_steps(0, T, np.zeros(B, np.int32))
    m.eval_end()
    torch.cuda.synchronize()
    e0.record(stream)
    reps = 3
    for _ in range(reps):
        m.decode_steps(0, T, np.zeros(B, np.int32))
        m.eval_end()
    e1.record(stream)
    torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / (reps * T)
    m.decoder_end()
    _, _, _, nfl = m.flat_buffers()
    m.close()
    peak_tf, peak_hbm, which, _ = peaks()
    step_bytes = decode_step_bytes(c, nfl)
    ach = step_bytes / (step_ms * 1e-3) / 1e9

    # (3) the file-level call a user makes: header parsing, payload upload, block walk, all segments
    ops = host.bind_cuda(p)
    t0 = time.perf_counter()
    back = host.decompress(ops, data, host.OUT_DEVICE)
    t_file = time.perf_counter() - t0
    host.unbind_cuda(ops)
    exact_file = bool(np.array_equal(back, toks))
    # and the walk on the host over trees copied back each step (what the device decoder replaces), 2 segments
    small = toks[: 2 * T * B]
    fp2 = host.file_params(p, block_len=small.size)
    ops = host.bind_cuda(p)
    d2, _ = host.compress(ops, fp2, small, host.EVAL_SEGMENT, host.OUT_CODER_READY)
    host.unbind_cuda(ops)
    ops = host.bind_cuda(p)
    t0 = time.perf_counter()
    back2 = host.decompress(ops, d2, host.OUT_CODER_READY)
    t_walk = time.perf_counter() - t0
    host.unbind_cuda(ops)
    exact_walk = bool(np.array_equal(back2, small))
    exact_parts = {"step_graphs": exact, "nch_decompress": exact_file, "host_walk": exact_walk}
    exact = exact and exact_file and exact_walk

    line = {"mode": "decode", "metric": "decoded symbols/s (one-symbol steps + train step per segment)",
            "value": value, "unit": "symbols/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms / K,
            "higher_is_better": True, "scaling": "replicas only", "vs_baseline": None,
            "dtype": "bf16" if p.use_bf16 else "f32", "data": "synthetic",
            "config": {"workload": workload_name(name, c).replace("train step", "decode (step mode) + train step"),
                       "tokens": "seeded Zipf(1.1)+order-1 Markov ids, encoded by this library's encoder first",
                       "l2": "the bf16 weights read by every step exceed the 126 MB L2" if 2 * nfl > 126e6 else
                             "the bf16 weights fit the 126 MB L2: DRAM traffic is below the algorithmic bytes"},
            "round_trip_exact": exact, "round_trip_exact_parts": exact_parts, "payload_bytes": len(payload), "payload_bytes_consumed": int(consumed),
            "bits_per_symbol": 8.0 * len(payload) / n, "gpu_launches": int(prof.launches), "clocks": clocks,
            "ms_per_symbol_step": step_ms,
            "e2e": {"value": n / t_file, "unit": "symbols/s", "h2d_bytes_per_step": B * 4 + T * B * 4,
                    "d2h_bytes_per_step": T * B * 4 + 4, "seconds": t_file,
                    "what": "nch_decompress over the whole file (bind excluded): payload upload, every segment, "
                            "symbols written to the host buffer"},
            "host_walk": {"value": small.size / t_walk, "unit": "symbols/s",
                          "what": "the same file format decoded with the trees copied to the host every step "
                                  "(nncu_coder_trees + nch_read_sym_tree), 2 segments"},
            "encode_symbols_per_s": n / t_enc,
            "roofline": {"bound": "hbm", "kernel": "one decode step (all kernels of the CUDA graph)", "achieved": ach,
                         "peak": peak_hbm, "unit": "GB/s", "frac": ach / peak_hbm, "traffic": None,
                         "peak_source": f"{which} hbm_gbs", "algorithmic_bytes_per_step": step_bytes}}
    print(json.dumps(line), flush=True)


def synth_prose(n_tokens, vocab=5000, seed=9):
    """Word soup with a Zipf law over `vocab` random lower-case words, capitals, all-caps, punctuation,
    doubled spaces and line ends: the shapes the case/space folding and the dictionary work on."""
    rng = np.random.default_rng(seed)
    words = [bytes(rng.integers(97, 123, rng.integers(1, 9)).astype(np.uint8)) for _ in range(vocab)]
    gaps = [b" ", b" ", b" ", b" ", b", ", b".\n", b"  ", b" (", b") ", b"-", b"", b"; "]
    pick, gap, style = rng.zipf(1.4, n_tokens) % vocab, rng.integers(0, len(gaps), n_tokens), rng.random(n_tokens)
    out = []
    for i in range(n_tokens):
        w = words[pick[i]]
        out += [w.capitalize() if style[i] < 0.12 else w.upper() if style[i] < 0.16 else w, gaps[gap[i]]]
    return b"".join(out)


def run_words(args):
    """The host pass in front of the model when text preprocessing is on: nch_words_encode (the
    restatement of the reference's word_encode) on synthetic prose, host cores only, with the
    reference's own stand-alone preprocessor timed on the same text where oracle/_ref holds it."""
    pkg = entry._package()
    H = pkg.host
    text = synth_prose(1_000_000)
    n_words, min_freq = 4096, 16
    times = []
    for _ in range(max(1, min(args.steps, 5))):
        t0 = time.perf_counter()
        d, syms, entries = H.words_encode(text, n_words, min_freq)
        times.append(time.perf_counter() - t0)
    t_enc = statistics.median(times)
    t0 = time.perf_counter()
    back = H.words_decode(d, syms)
    t_dec = time.perf_counter() - t0
    base = None
    from oracle import oracle as orc
    exe = orc.preprocess_ref()
    if exe and not args.no_cpu_baseline:
        import tempfile
        with tempfile.TemporaryDirectory() as td:
            f = {k: os.path.join(td, k) for k in ("in", "dict", "sym")}
            open(f["in"], "wb").write(text)
            t0 = time.perf_counter()
            subprocess.run([exe, "c", f["dict"], f["in"], f["sym"], str(n_words), str(min_freq)], check=True,
                           capture_output=True, timeout=600)
            t_ref = time.perf_counter() - t0
            same = open(f["dict"], "rb").read() == d and open(f["sym"], "rb").read() == syms.astype(">u2").tobytes()
        base = {"value": len(text) / t_ref, "unit": "bytes/s", "cores": 1, "kind": "reference",
                "sample": "the same text through the reference's stand-alone preprocess tool (file to file)",
                "same_output": bool(same)}
    print(json.dumps({"metric": "tokenizer_text_bytes_per_second", "value": len(text) / t_enc, "unit": "bytes/s",
                      "n_gpus": 0, "steps": len(times), "higher_is_better": True, "dtype": "u16", "data": "synthetic",
                      "config": {"workload": f"word tokenizer, {len(text)} bytes of synthetic prose, n_words {n_words}, "
                                             f"min_freq {min_freq}", "entries": entries, "symbols": int(syms.size)},
                      "symbols_per_second": syms.size / t_enc, "decode_bytes_per_second": len(text) / t_dec,
                      "round_trip_exact": back == text, "cores": 1, "cpu_baseline": base}))


def profile_traffic(kernel_md):
    """`traffic_bytes_per_launch: <number>` from a profile summary under profiles/ (ncu's
    dram__bytes_read.sum + dram__bytes_write.sum per launch), or None."""
    try:
        text = open(os.path.join(ROOT, "profiles", kernel_md)).read()
    except OSError:
        return None
    mt = re.search(r"traffic_bytes_per_launch:\s*([0-9.eE+]+)", text)
    return float(mt.group(1)) if mt else None


def attention_record(pkg, lib, torch, peak_tf_burst, peak_hbm, which, reps=120):
    """BASELINE config[1]: the isolated relative-position attention op, 16 streams x 8 heads x
    d_head 64, 64 queries over 64 + 64 keys, R of length 128, bf16, forward and backward through
    the C ABI.  Twelve operand sets are used in rotation (12 x 12.7 MB > the 126 MB L2), so every
    call reads its operands from HBM."""
    B, H, dk, T, M, P = 16, 8, 64, 64, 64, 128
    L, HD = M + T, H * dk
    nsets = 12
    g = torch.Generator(device="cpu").manual_seed(7)
    bf = torch.bfloat16
    mk = lambda *sh: torch.randn(nsets, *sh, generator=g).to(bf).cuda()
    q, kv, dout = mk(T * B, HD), mk(L * B, 2 * HD), mk(T * B, HD)
    out, dq, dkv = torch.zeros_like(q), torch.zeros_like(q), torch.zeros_like(kv)
    lse = torch.zeros(nsets, B * H, T, device="cuda")
    w_r = (0.02 * torch.randn(H, P, dk, generator=g)).cuda()
    b_r = (0.02 * torch.randn(H, L, generator=g)).cuda()
    pw, pb = torch.zeros(B, H, P, dk, device="cuda"), torch.zeros(B, H, L, device="cuda")
    gw, gb = torch.zeros(H, P, dk, device="cuda"), torch.zeros(H, L, device="cuda")
    shp = pkg.abi.AttnShape(B, H, dk, T, M, P, 0, 0, T, float(np.sqrt(dk * 512.0)), 1)
    st = torch.cuda.current_stream()
    sp = C.c_void_p(st.cuda_stream)

    def ck(rc):
        if rc != 0:
            raise RuntimeError(lib.nncu_last_error().decode())

    def fwd(i):
        ck(lib.nncu_attention_forward(C.byref(shp), q[i].data_ptr(), kv[i].data_ptr(), w_r.data_ptr(),
                                      b_r.data_ptr(), out[i].data_ptr(), lse[i].data_ptr(), sp))

    def bwd(i):
        ck(lib.nncu_attention_backward(C.byref(shp), q[i].data_ptr(), kv[i].data_ptr(), w_r.data_ptr(),
                                       b_r.data_ptr(), out[i].data_ptr(), lse[i].data_ptr(), dout[i].data_ptr(),
                                       dq[i].data_ptr(), dkv[i].data_ptr(), pw.data_ptr(), pb.data_ptr(), sp))
        ck(lib.nncu_attention_reduce_tables(C.byref(shp), pw.data_ptr(), pb.data_ptr(), gw.data_ptr(),
                                            gb.data_ptr(), 0, sp))

    def timed(body):
        """Average device time of body(i) over `reps` calls that walk the operand sets: the calls of
        one walk are captured into a CUDA graph (the library launches on torch's current stream) and
        the graph is replayed, so the figure is GPU time, not the Python launch rate."""
        for i in range(nsets):
            body(i)        # eager first: kernel attributes, tensor maps, per-device set-up
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            sp.value = side.cuda_stream
            with torch.cuda.graph(graph, stream=side):
                for i in range(nsets):
                    body(i)
            walks = max(1, reps // nsets)
            graph.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            for r in range(walks):
                graph.replay()
            e1.record(side)
            side.synchronize()
        sp.value = st.cuda_stream
        return e0.elapsed_time(e1) * 1e-3 / (walks * nsets)

    t_f = timed(fwd)
    t_fb = timed(lambda i: (fwd(i), bwd(i)))
    fam = 2.0 * B * H * T * L * dk
    fl_f, fl_fb = 3 * fam, 11 * fam          # QK^T, W_r^T q, PV; the backward recomputes both score products
    byt = 2.0 * (4 * T * B * HD + 4 * L * B * HD) + 4.0 * (H * P * dk + H * L)
    floor_f = max(fl_f / (peak_tf_burst * 1e12), 2.0 * (2 * T * B * HD + 2 * L * B * HD) / (peak_hbm * 1e9))
    floor_fb = max(fl_fb / (peak_tf_burst * 1e12), byt / (peak_hbm * 1e9))
    return {"config": "BASELINE config[1]: 16 streams x 8 heads x d_head 64, 64 queries, 64+64 keys, R length 128, "
                      "bf16 operands, fp32 accumulation; 12 operand sets in rotation (working set > L2)",
            "reps": max(1, reps // nsets) * nsets, "timing": "CUDA-graph replay of one walk over the operand sets, CUDA events", "fwd_us": t_f * 1e6, "fwd_bwd_us": t_fb * 1e6,
            "fwd_tflops": fl_f / t_f / 1e12, "fwd_bwd_tflops": fl_fb / t_fb / 1e12,
            "fwd_gflop": fl_f / 1e9, "fwd_bwd_gflop": fl_fb / 1e9,
            "flops_counted": "forward 3 contraction families, backward 8 (both score products recomputed)",
            "roofline": {"bound": "min(tensor, hbm): hbm", "floor_us_fwd": floor_f * 1e6,
                         "floor_us_fwd_bwd": floor_fb * 1e6, "frac_fwd": floor_f / t_f,
                         "frac_fwd_bwd": floor_fb / t_fb, "operand_bytes_fwd_bwd": byt,
                         "peak_source": f"{which} bf16_tflops (burst) and hbm_gbs"}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--config", default=None, choices=sorted(CONFIGS), help="default: c2 (train), c4 (decode)")
    ap.add_argument("--mode", default="train", choices=["train", "decode", "words"])
    ap.add_argument("--backend", type=int, default=0, help="0 auto, 1 SIMT, 2 tcgen05")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-attention", action="store_true", help="skip the config[1] attention record")
    ap.add_argument("--repeats", type=int, default=7, help="times the K-step region is measured (median reported)")
    args = ap.parse_args()
    if args.mode == "words":
        run_words(args)
        return
    if args.config is None:
        args.config = "c4" if args.mode == "decode" else "c2"
    c = dict(CONFIGS[args.config])
    if args.mode == "decode" and args.impl != "reference":
        if args.steps == 100:
            args.steps = 8
        run_decode(args, c, args.config)
        return
    if args.impl == "reference":
        run_reference(args, c)
        return

    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local)
    if world > 1:
        # the library pins NCCL's algorithm, protocol and channel count when its communicator is made;
        # NCCL reads some of them once per process, so they go in before torch's communicator exists
        if os.environ.get("NNCU_NCCL_PIN") != "0":
            for k, v in (("NCCL_ALGO", "Ring"), ("NCCL_PROTO", "LL128"), ("NCCL_MIN_NCHANNELS", "32"),
                         ("NCCL_MAX_NCHANNELS", "32")):
                os.environ.setdefault(k, v)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = entry._package()
    lib = pkg.library()   # raises if the CUDA library is not built: there is no other path

    Bt = c["n_streams"]
    if Bt % world:
        raise SystemExit("streams must divide over the ranks")
    B = Bt // world
    kw = dict(COMMON)
    kw.update(c)
    kw.update(n_streams=B, n_streams_total=Bt, gemm_backend=args.backend, device=local)
    p = pkg.abi.make_params(**kw)
    m = pkg.TrfModel(p)
    # a non-default stream: the library then replays CUDA graphs of forward and backward
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    m.set_stream(stream.cuda_stream)
    T, V = c["seg_len"], c["n_symbols"]
    K, W = args.steps, max(args.warmup, 3)
    REPEATS = max(1, args.repeats)
    ids_all, tg_all = make_batches(c, Bt, K + W)
    sl = pkg.dist.stream_slice(rank, world, Bt)
    ids_h = torch.from_numpy(np.ascontiguousarray(ids_all[:, :, sl])).pin_memory()
    tg_h = torch.from_numpy(np.ascontiguousarray(tg_all[:, :, sl])).pin_memory()
    ids_d, tg_d = ids_h.cuda(), tg_h.cuda()

    wptr, gptr, vptr, nfl = m.flat_buffers()
    # the flat gradient buffer as a torch tensor (for the NCCL all-reduce)
    grads = torch.as_tensor(pkg.dist.CudaArray(gptr, nfl), device=f"cuda:{local}") if world > 1 else None
    if world > 1 and os.environ.get("NNCU_PY_ALLREDUCE") != "1":
        # per-layer all-reduces inside the backward pass instead of one all-reduce after it
        pkg.dist.attach_library_comm(m, lib, rank, world, torch.device("cuda", local))
    sharded = pkg.dist.ShardedStep(m, grads, world=world)

    def step_device(s):
        sharded.step_device(ids_d[s].data_ptr(), tg_d[s].data_ptr())
        if world > 1:
            # read the segment's loss (as a host would): it keeps the ranks' hosts within one step
            # of their GPUs.  With 50 steps queued ahead the ranks drift apart and each NCCL kernel
            # spins on SMs until its peer arrives: measured 360-770 k symbols/s from run to run at
            # 2 GPUs, against a steady 800 k with this read.
            m.read_loss()

    nb = int(np.log2(V)) if (V & (V - 1)) == 0 else 0
    paths = np.zeros((T * B, max(nb, 1)), np.uint16)
    nbits = C.c_int()

    def step_host(s, last=True):
        # encoder order: everything is queued before the host waits for anything, so the GPU
        # never idles on the host (the range coder would run between _begin and _end).  An encoder
        # knows the next segment's symbols too: its forward pass is queued (last=False) before the host
        # waits for this segment's coder values and loss.
        ids, tg = ids_h[s].numpy(), tg_h[s].numpy()
        if not step_host.queued:
            m.eval(-1, ids, read=False)
        step_host.queued = False
        if nb:
            ck(lib.nncu_coder_paths_begin(m.h, 0, T, tg.ctypes.data_as(C.c_void_p)))
        else:
            m.read_probs(0, T)
        if sharded.fused():
            ck(lib.nncu_eval_gradient_update(m.h, tg.ctypes.data_as(C.c_void_p), None))
            m.memory_shift()
        else:
            ck(lib.nncu_eval_gradient(m.h, tg.ctypes.data_as(C.c_void_p), None))
            sharded.reduce_gradients()
            m.update()
        if not last:
            m.eval(-1, ids_h[s + 1].numpy(), read=False)
            step_host.queued = True
        if nb:
            ck(lib.nncu_coder_paths_end(m.h, paths.ctypes.data_as(C.c_void_p), C.byref(nbits)))
        return m.read_loss()

    step_host.queued = False

    def ck(rc):
        if rc != 0:
            raise RuntimeError(lib.nncu_last_error().decode())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # Initialisation, not warm-up: the library captures its CUDA graphs on the second use of each
    # memory twin (four steps), and NCCL sets its channels up on the first collectives.  Without
    # these steps a 3-step warm-up leaves both inside the timed region (seen at 2 GPUs as run-to-run
    # swings of the device-resident figure between 360 k and 770 k symbols/s).
    m.reset()
    for s in range(6):
        step_device(s % (W + K))
    barrier()
    m.reset()
    for s in range(W):
        step_device(s)
    barrier()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()
        return ms

    # the K-step region, REPEATS times; each repeat bracketed by barrier + synchronize
    times = []
    launches = 0
    for r in range(REPEATS):
        barrier()
        lib.nncu_profile_begin(0)
        e0.record(stream)
        for s in range(W, W + K):
            step_device(s)
        e1.record(stream)
        barrier()
        prof = pkg.abi.Profile()
        lib.nncu_profile_end(C.byref(prof))
        launches = int(prof.launches)
        times.append(max_over_ranks(e0.elapsed_time(e1)))
    m.synchronize()
    ms = statistics.median(times)
    value = K * T * Bt / (ms * 1e-3)

    # end to end through the host-buffer calls
    m.reset()
    for s in range(2):
        step_host(s)
    times_e2e = []
    for r in range(REPEATS):
        barrier()
        t0 = time.perf_counter()
        e0.record(stream)
        for s in range(W, W + K):
            step_host(s, last=(s == W + K - 1))
        e1.record(stream)
        barrier()
        times_e2e.append(max_over_ranks(max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3)))
    clocks = sampler.stop() if sampler else None   # sampled over both timed regions
    ms_e2e = statistics.median(times_e2e)
    e2e = K * T * Bt / (ms_e2e * 1e-3)

    # per-launch timing of the dominant kernel (separate short pass so the timed region above
    # carries no event overhead)
    roof = None
    peak_tf, peak_hbm, which, peak_tf_burst = peaks()
    if p.use_bf16 and args.backend != 1:
        lib.nncu_profile_begin(1)
        for s in range(W, W + min(K, 3)):
            step_device(s)
        barrier()
        pr = pkg.abi.Profile()
        lib.nncu_profile_end(C.byref(pr))
        if pr.gemm_launches:
            ach = pr.gemm_flops / (pr.gemm_ms * 1e-3) / 1e12
            traffic = profile_traffic("gemm_tc_kernel_c2_dram_traffic.md") if (args.config == "c2" and world == 1) else None
            roof = {"bound": "tensor", "kernel": "gemm_tc_kernel (tcgen05 bf16 GEMM, all operand arrangements)",
                    "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
                    "peak_source": f"{which} bf16_tflops_sustained",
                    "traffic": traffic,
                    "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum per launch, from the committed "
                                      "profile summary of this kernel on this workload (not re-measured by this run)",
                    "launches_per_step": pr.gemm_launches / min(K, 3),
                    "share_of_step": (pr.gemm_ms / min(K, 3)) / (ms / K)}
    attn = None
    if rank == 0 and not args.no_attention:
        attn = attention_record(pkg, lib, torch, peak_tf_burst, peak_hbm, which)
    m.synchronize()
    whash = m.weights_hash()
    if world > 1:
        hs = [None] * world
        dist.all_gather_object(hs, whash)
        same = len(set(hs)) == 1
    else:
        same = True

    if rank == 0:
        fl = step_flops(dict(c, ff_act=COMMON["ff_act"]), Bt)
        line = {"metric": "compressed symbols/s (fwd+bwd+RMSProp)", "value": value, "unit": "symbols/s",
                "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if p.use_bf16 else "f32",
                "data": "synthetic",
                "config": job_config(args.config, c, world, exchange_name(world) if (world == 1 or m.has_comm)
                                     else "one all-reduce after backward"),
                "repeats": REPEATS, "value_min": K * T * Bt / (max(times) * 1e-3),
                "value_max": K * T * Bt / (min(times) * 1e-3),
                "step_tflops": fl / (ms / K * 1e-3) / 1e12, "step_gflop": fl / 1e9,
                "gpu_launches": launches, "clocks": clocks,
                "e2e": {"value": e2e, "unit": "symbols/s", "h2d_bytes_per_step": 2 * T * B * 4 * world,
                        "d2h_bytes_per_step": (T * B * nb * 2 + 4) * world if nb else (T * B * V * 4 + 4) * world,
                        "ms_per_step": ms_e2e / K, "value_min": K * T * Bt / (max(times_e2e) * 1e-3),
                        "value_max": K * T * Bt / (min(times_e2e) * 1e-3)},
                "ranks_hold_identical_weights": same, "weights_hash": f"{whash:016x}"}
        if roof:
            line["roofline"] = roof
        if attn:
            line["attention"] = attn
        if not args.no_cpu_baseline and world == 1:
            streams = CPU_STREAMS.get(args.config, c["n_streams"])
            val, dt, threads = cpu_port_run(c, 6, 1, streams)
            line["cpu_baseline"] = {"value": val, "unit": "symbols/s", "cores": threads, "kind": "port",
                                    "sample": f"6 steps of {streams} of the {c['n_streams']} streams x {T} symbols "
                                              f"of the same model (oracle/trf_oracle.c, OpenMP on {threads} "
                                              f"threads, {dt:.1f} s)"}
        print(json.dumps(line), flush=True)
    barrier()
    m.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    sys.stdout.flush()


if __name__ == "__main__":
    main()
