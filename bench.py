#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with roofline fractions.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the SmolLM2-1.7B shape (24 layers, hidden 2048, 32/32 heads, head size
64, SwiGLU 8192, vocabulary 49152, tied embeddings), random N(0, 0.02) bfloat16 weights,
synthetic prompt ids uniform over the vocabulary; batch of 8 requests decoding at a
2,048-token context.  A "step" is one decode step of the whole batch.  Prints ONE JSON line:

  value        decoded tokens per second, timed on the device with CUDA events
  e2e          the same through the Python entry point (Engine.step): host tokens in from
               pinned memory, sampled tokens read back to the host, every step
  prefill      one step of 2,048 prompt tokens; frac = flops / time / bf16 peak (float32 runs:
               / the float32 peak of the CUDA cores)
  roofline     decode step: bytes it must read (every weight once + the cache of the live
               requests) / time, against the copy bandwidth
  points       decode tokens per second at batch 1 and 64
  fp32         decode and prefill of the same shape on the true 32-bit path

Other workloads: --shape smollm2-360m|llama3-8b runs the same measurements on those layer
sizes; --workload serve pushes 64 mixed requests through the engine's scheduler under a
512-token budget and reports generated tokens per second by the host clock.

Peaks come from MEASURED_PEAKS.json beside this file when present ("of measured"), else
from the fallback figures of an earlier measurement on this kind of GPU ("of fallback").
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
# The like-for-like baseline: tkran2/bitwise's Runner::forward on the SmolLM2-1.7B shape, 8 threads on
# this image's CPU, 2,048-token contexts, as BASELINE.md records it (decode tokens per second by batch).
# The reference publishes no figure for this batch and context (its README has 7.26 tok/s single stream).
BASELINE_DECODE_TOKS = {("smollm2-1.7b", 2048, 1): 10.7, ("smollm2-1.7b", 2048, 8): 29.9, ("smollm2-1.7b", 2048, 64): 35.4}
REFERENCE_SOURCE = "/root/reference"


def fp32_simt_tflops():
    """The float32 peak of the CUDA cores, from the device's own figures: SMs x 128 lanes x 2
    flops x the highest SM clock (what the true 32-bit path, which uses no tensor core, is
    measured against)."""
    import torch
    props = torch.cuda.get_device_properties(0)
    mhz = 0.0
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits", "-i", "0"],
                             capture_output=True, text=True, timeout=10).stdout.strip().splitlines()
        mhz = float(out[0])
    except Exception:
        mhz = 0.0
    if mhz <= 0:
        mhz = 1965.0
    return props.multi_processor_count * 128 * 2 * mhz * 1e6 / 1e12


def peaks():
    path = os.path.join(HERE, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            d = json.load(open(path))
            flat = {}

            def walk(x):
                if isinstance(x, dict):
                    for k, v in x.items():
                        if isinstance(v, (int, float)):
                            flat.setdefault(k, float(v))
                        else:
                            walk(v)
            walk(d)
            hbm = flat.get("hbm_gbs")
            tf = flat.get("bf16_tflops")
            tfs = flat.get("bf16_tflops_sustained", tf)
            if hbm and tf:
                return dict(hbm_gbs=hbm, bf16_tflops=tf, bf16_tflops_sustained=tfs, source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, bf16_tflops_sustained=1400.0,
                source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                          "-i", "0", "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            p = [x.strip() for x in line.split(",")]
            if len(p) >= 6 and p[0].isdigit():
                self.samples.append(p)

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        mhz = sorted(int(s[0]) for s in self.samples)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons,
                "samples": len(mhz)}


SHAPES = {
    # name: (title, layers, LlamaConfig keywords, default decode context)
    "smollm2-1.7b": ("SmolLM2-1.7B shape", 24, dict(
        vocab_size=49152, hidden_size=2048, num_attention_heads=32, num_key_value_heads=32, head_dim=64,
        intermediate_size=8192, rope_theta=130000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
        max_position_embeddings=8192), 2048),
    "smollm2-360m": ("SmolLM2-360M shape", 32, dict(
        vocab_size=49152, hidden_size=960, num_attention_heads=15, num_key_value_heads=5, head_dim=64,
        intermediate_size=2560, rope_theta=100000.0, rms_norm_eps=1e-5, tie_word_embeddings=True,
        max_position_embeddings=8192), 2048),
    "llama3-8b": ("Llama-3-8B shape", 32, dict(
        vocab_size=128256, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
        intermediate_size=14336, rope_theta=500000.0, rms_norm_eps=1e-5, tie_word_embeddings=False,
        max_position_embeddings=8192,
        rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                          original_max_position_embeddings=8192)), 4096),
}


def model_config(shape, layers):
    from bitwise_b200 import LlamaConfig
    from bitwise_b200.config.llama import RopeScaling
    kw = dict(SHAPES[shape][2])
    if "rope_scaling" in kw:
        kw["rope_scaling"] = RopeScaling(**kw["rope_scaling"])
    return LlamaConfig(num_hidden_layers=layers, **kw)


def matrix_params(c):
    per_layer = (c.q_dim + 2 * c.kv_dim) * c.hidden_size + c.hidden_size * c.q_dim + 3 * c.hidden_size * c.intermediate_size
    return per_layer * c.num_hidden_layers, c.vocab_size * c.hidden_size


def decode_bytes(c, batch, ctx, elt):
    body, head = matrix_params(c)
    kv = batch * ctx * c.num_hidden_layers * 2 * c.kv_dim * elt
    return (body + head) * elt + kv + batch * c.hidden_size * elt


def prefill_flops(c, tokens):
    body, head = matrix_params(c)
    attn = c.num_hidden_layers * 2 * 2 * c.q_dim * (tokens * (tokens + 1) // 2)
    return 2.0 * tokens * body + 2.0 * head + attn


def run_decode(model, batch, ctx, steps, warmup, page, seed=0):
    """Device-timed decode: `batch` requests, each with `ctx` tokens in the cache, one new
    token each per step, sampled greedily on the device."""
    import numpy as np
    import torch
    from bitwise_b200.cache.storage import build_cache
    from bitwise_b200.engine.step import StepEntry, Stepper
    c = model.config
    total = ctx + warmup + steps + 1
    pages_per = (total + page - 1) // page
    manager, storage = build_cache(model.decoder, pages_per * batch, page, batch, torch.bfloat16 if
                                   model.dtype == "bfloat16" else torch.float32, model.device)
    chunk = 2048
    st = Stepper(model.decoder, manager, storage, model.ops, max_rows=max(chunk, batch), max_seqs=batch,
                 max_tokens_per_request=pages_per * page)
    rng = np.random.default_rng(seed)
    for b in range(batch):  # fill the contexts by real prefill
        toks = rng.integers(0, c.vocab_size, ctx - 1).tolist()
        for i in range(0, len(toks), chunk):
            st.run([StepEntry(b, toks[i:i + chunk], [])])
    nxt = rng.integers(0, c.vocab_size, batch).tolist()
    temps = torch.zeros(batch, device=model.device)
    us = torch.zeros(batch, dtype=torch.float64, device=model.device)
    out = torch.zeros(batch, dtype=torch.int32, device=model.device)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def one_step():
        logits = st.run([StepEntry(b, [nxt[b]], [0]) for b in range(batch)])
        model.ops.sample_rows(logits, temps, us, out)

    for _ in range(warmup):
        one_step()
    torch.cuda.synchronize()
    l0 = model.ops.launches
    ev0.record()
    for _ in range(steps):
        one_step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    launches = model.ops.launches - l0
    del st, manager, storage
    torch.cuda.empty_cache()
    return ms, launches


def run_prefill(model, tokens, reps, warmup, page):
    import numpy as np
    import torch
    from bitwise_b200.cache.storage import build_cache
    from bitwise_b200.engine.step import StepEntry, Stepper
    c = model.config
    pages = (tokens + page - 1) // page
    manager, storage = build_cache(model.decoder, pages, page, 1, torch.bfloat16 if model.dtype == "bfloat16"
                                   else torch.float32, model.device)
    st = Stepper(model.decoder, manager, storage, model.ops, max_rows=tokens, max_seqs=1,
                 max_tokens_per_request=pages * page)
    toks = np.random.default_rng(1).integers(0, c.vocab_size, tokens).tolist()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(warmup + reps):
        torch.cuda.synchronize()
        ev0.record()
        st.run([StepEntry("p", toks, [tokens - 1])])
        ev1.record()
        torch.cuda.synchronize()
        st.finish("p")
        if i >= warmup:
            times.append(ev0.elapsed_time(ev1))
    del st, manager, storage
    torch.cuda.empty_cache()
    return sorted(times)[len(times) // 2]


def run_e2e(model, batch, ctx, steps, warmup, page, fingerprint=True):
    """Through Engine.step(): prompts of ctx-1 tokens are prefilled by the engine itself, then
    `steps` decode steps are timed by the host clock, each with its host-to-device copy of the
    step's inputs and the device-to-host read of the sampled tokens.  ``fingerprint``: the
    engine's default, a hash of every sampled row's logits chained on the device."""
    import numpy as np
    import torch
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    c = model.config
    total = ctx + warmup + steps + batch + 16
    pages_per = (total + page - 1) // page
    eng = Engine(model, EngineConfig(num_blocks=pages_per * batch, block_size=page, max_batched_tokens=2048,
                                     max_num_seqs=batch, fingerprint_logits=fingerprint,
                                     max_model_len=pages_per * page))
    rng = np.random.default_rng(2)
    sp = SamplingParams(temperature=0.0, max_new_tokens=warmup + steps + batch + 8, ignore_eos=True)
    for b in range(batch):
        eng.add_request(rng.integers(0, c.vocab_size, ctx - 1).tolist(), sp)
    guard = 0
    while eng.stats.prefill_tokens < batch * (ctx - 1):  # until every request has left its prompt behind
        eng.step()
        guard += 1
        assert guard < 10000
    for _ in range(max(warmup, 3)):  # decode steps only from here on; the first ones build the step's graph
        eng.step()
    torch.cuda.synchronize()
    g0 = eng.stats.generated_tokens
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    made = eng.stats.generated_tokens - g0
    h2d = eng.stepper.h2d_bytes + eng._samp_host.numel()
    d2h = eng.d2h_bytes
    del eng
    torch.cuda.empty_cache()
    return made / dt, h2d, d2h


# ---- the Nuderax design beside Llama at equal size (--compare nuderax) -------------------------
NUDERAX_SIZES = {
    # width, layers run, heads, dim, rot_dim, vdim, kv_rank, q_rank, experts, groups, keep, top, ff, shared ff, vocab
    "small": dict(width=1024, layers=4, heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=512, experts=16,
                  groups=4, keep=2, top=2, ff=512, shared_ff=1024, vocab=32768),
    "medium": dict(width=2048, layers=4, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=1024, experts=64,
                   groups=8, keep=4, top=6, ff=1408, shared_ff=2816, vocab=32768),
}


def nuderax_config(z):
    from bitwise_b200.config import LatentMixerConfig, NuderaxConfig, NuderaxLayerConfig, RoutedMlpConfig
    layers = []
    for i in range(z["layers"]):
        kind = "latent_attention_2" if i % 2 == 0 else "latent_attention"
        m = LatentMixerConfig(kind, z["heads"], z["dim"], z["rot_dim"], z["vdim"], z["kv_rank"],
                              (z["dim"] + z["rot_dim"]) ** -0.5, 10000.0, z["rot_dim"],
                              z["q_rank"] if kind == "latent_attention_2" else None, None)
        f = RoutedMlpConfig(z["experts"], z["top"], 1.0, z["groups"], z["keep"], z["ff"], 7.0, z["shared_ff"], 7.0)
        layers.append(NuderaxLayerConfig(m, f))
    return NuderaxConfig(vocab=z["vocab"], width=z["width"], eps=1e-5, layers=tuple(layers))


def llama_twin(z):
    """Llama with the same width, layers, heads and vocabulary, a head of dim + rot_dim, and the
    feed-forward width a token of the routed model is multiplied with (top experts and the shared one)."""
    from bitwise_b200 import LlamaConfig
    return LlamaConfig(vocab_size=z["vocab"], hidden_size=z["width"], num_hidden_layers=z["layers"],
                       num_attention_heads=z["heads"], num_key_value_heads=z["heads"], head_dim=z["vdim"],
                       intermediate_size=(z["top"] * z["ff"] + z["shared_ff"]) // 64 * 64, rope_theta=10000.0,
                       rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=8192)


class KernelBatch:
    """A step's index arrays for timing a kernel alone: ``seqs`` = [(first position, rows)]."""

    def __init__(self, seqs, heights, device, granule=256):
        import torch
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
        pos, row_seq, p0s, r0s = [], [], [], []
        r = 0
        for s, (p0, cnt) in enumerate(seqs):
            p0s.append(p0), r0s.append(r)
            pos += list(range(p0, p0 + cnt))
            row_seq += [s] * cnt
            r += cnt
        self.n, self.num_seqs = r, len(seqs)
        self.pos, self.row_seq, self.seq_pos0, self.seq_row0 = i32(pos), i32(row_seq), i32(p0s), i32(r0s + [r])
        self.max_keys = (max(pos) + 1 + granule - 1) // granule * granule
        self.tile_sets = {}
        for h in heights:
            listed = []
            for s, (p0, cnt) in enumerate(seqs):
                for a in range(0, cnt, h):
                    rows = min(h, cnt - a)
                    listed.append((-(p0 + a + rows), s, r0s[s] + a, rows))
            listed.sort()
            self.tile_sets[h] = (i32([x[1] for x in listed]), i32([x[2] for x in listed]), i32([x[3] for x in listed]),
                                 len(listed))

    def query_tiles(self, h):
        return self.tile_sets[h]


def timed(fn, reps=7, flush=None):
    """Median device time in ms of ``fn`` (CUDA events on the launching stream); ``flush`` is
    written before every repetition so that nothing of the last one stays in L2."""
    import torch
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for i in range(reps + 3):
        if flush is not None:
            flush.zero_()
        torch.cuda.synchronize()
        ev0.record()
        fn()
        ev1.record()
        torch.cuda.synchronize()
        if i >= 3:
            times.append(ev0.elapsed_time(ev1))
    return sorted(times)[len(times) // 2]


def timed_device(fn, reps=7, flush=None):
    """Median device time in ms of the kernels that ``fn`` launches: they are captured into a CUDA
    graph once and the replay is timed, so that the host's share of a call (argument checks of a
    binding take longer than a small kernel runs) stays out of the figure."""
    import torch
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return timed(graph.replay, reps=reps, flush=flush)


def kernel_table(z, pk, page=16):
    """Every new kernel alone at the size's shapes beside the like kernel of the Llama twin:
    milliseconds and the fraction of its roofline (measured copy bandwidth or bf16 peak)."""
    import torch
    from bitwise_b200.kernels.ops import get_ops
    ops = get_ops("bfloat16")
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, rank, rot, dim, vdim, width = z["heads"], z["kv_rank"], z["rot_dim"], z["dim"], z["vdim"], z["width"]
    dk = rank + rot
    hd = vdim
    out = {}

    def frac_flops(flops, ms):
        return round(flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"], 4)

    def frac_bytes(nbytes, ms):
        return round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    def put(name, ms, frac, twin_ms, twin_frac, bound):
        out[name] = {"ms": round(ms, 4), "frac": frac, "twin_ms": round(twin_ms, 4), "twin_frac": twin_frac, "bound": bound,
                     "gap_ratio": round(twin_frac / frac, 2) if frac else None}

    for label, seqs in (("prefill_2048", [(0, 2048)]), ("decode_b8_ctx2048", [(2047, 1)] * 8)):
        keys = max(p0 + c for p0, c in seqs)
        blocks = (keys + page - 1) // page
        nseq = len(seqs)
        table = torch.arange(nseq * blocks, dtype=torch.int32, device=dev).reshape(nseq, blocks)
        heights = set(ops.latent_attention_tile_heights(H, rank, rot)) | set(ops.attention_tile_heights(H, H, hd))
        b = KernelBatch(seqs, sorted(heights), dev)
        n = b.n
        pairs = sum(c * p0 + c * (c + 1) // 2 for p0, c in seqs)
        # latent attention
        cache = torch.randn(nseq * blocks + 1, page, dk, device=dev).to(bf)
        q = torch.randn(n, H * dk, device=dev).to(bf)
        o = torch.empty(n, H * rank, dtype=bf, device=dev)
        ms = timed(lambda: ops.latent_attention(q, cache, table, o, H, rank, rot, dk ** -0.5, b), flush=flush)
        # the Llama twin's attention
        kc = torch.randn(nseq * blocks + 1, H, page, hd, device=dev).to(bf)
        vc = torch.randn(nseq * blocks + 1, H, page, hd, device=dev).to(bf)
        qkv = torch.randn(n, 3 * H * hd, device=dev).to(bf)
        o2 = torch.empty(n, H * hd, dtype=bf, device=dev)
        tms = timed(lambda: ops.attention(qkv, kc, vc, table, b.row_seq, b.pos, o2, H, H, hd, 0, b.max_keys, hd ** -0.5,
                                          batch=b), flush=flush)
        if n > nseq:
            put(f"attention_{label}", ms, frac_flops(2.0 * H * (dk + rank) * pairs, ms), tms,
                frac_flops(4.0 * H * hd * pairs, tms), "bf16 peak")
        else:
            put(f"attention_{label}", ms, frac_bytes(nseq * keys * dk * 2, ms), tms, frac_bytes(nseq * keys * 2 * H * hd * 2, tms),
                "copy bandwidth")
        # the experts' products against the twin's dense ones
        E, top, ff = z["experts"], z["top"], z["ff"]
        inter = (top * ff + z["shared_ff"]) // 64 * 64
        x = torch.randn(n, width, device=dev).to(bf)
        chosen = torch.stack([torch.randperm(E, device=dev)[:top] for _ in range(n)]).to(torch.int32)
        lists = torch.empty(3, E + 1, dtype=torch.int32, device=dev)
        order = torch.empty(n * top, dtype=torch.int32, device=dev)
        place = torch.empty(n * top, dtype=torch.int32, device=dev)
        ops.group_rows(chosen, E, lists[0], lists[1:3], order, place)
        w1 = (torch.randn(E, 2 * ff, width, device=dev) * 0.02).to(bf)
        w2 = (torch.randn(E, width, ff, device=dev) * 0.02).to(bf)
        gu = torch.empty(n * top, 2 * ff, dtype=bf, device=dev)
        hh = torch.randn(n * top, ff, device=dev).to(bf)
        y = torch.empty(n * top, width, dtype=torch.float32, device=dev)
        grouped = (lists[0], lists[1:3], order)
        xs = torch.empty(n * top, width, dtype=bf, device=dev)
        ms1 = timed(lambda: ops.grouped_linear(x, w1, gu, n * top, lists=grouped, order_div=top, sorted_x=xs), flush=flush)
        ms2 = timed(lambda: ops.grouped_linear(hh, w2, y, n * top, lists=grouped, gather=False), flush=flush)
        wd1 = (torch.randn(2 * inter, width, device=dev) * 0.02).to(bf)
        wd2 = (torch.randn(width, inter, device=dev) * 0.02).to(bf)
        g2 = torch.empty(n, 2 * inter, dtype=bf, device=dev)
        h2 = torch.randn(n, inter, device=dev).to(bf)
        y2 = torch.zeros(n, width, dtype=torch.float32, device=dev)
        t1 = timed(lambda: ops.linear(x, wd1, g2), flush=flush)
        t2 = timed(lambda: ops.linear(h2, wd2, y2, residual=y2), flush=flush)
        used = min(E, n * top) if n * top < 4 * E else E  # experts whose weights a step reads (about)
        if n > nseq:
            put(f"experts_gate_up_{label}", ms1, frac_flops(2.0 * n * top * 2 * ff * width, ms1), t1,
                frac_flops(2.0 * n * 2 * inter * width, t1), "bf16 peak")
            put(f"experts_down_{label}", ms2, frac_flops(2.0 * n * top * ff * width, ms2), t2,
                frac_flops(2.0 * n * inter * width, t2), "bf16 peak")
        else:
            used = int(torch.unique(chosen).numel())
            put(f"experts_gate_up_{label}", ms1, frac_bytes(used * 2 * ff * width * 2, ms1), t1,
                frac_bytes(2 * inter * width * 2, t1), "copy bandwidth")
            put(f"experts_down_{label}", ms2, frac_bytes(used * ff * width * 2, ms2), t2, frac_bytes(inter * width * 2, t2),
                "copy bandwidth")
        # the products per head around attention (no twin: Llama has none), the norms, the routing
        qh = torch.randn(n, H * (dim + rot), device=dev).to(bf)
        wk = (torch.randn(H, rank, dim, device=dev) * 0.05).to(bf)
        qf = torch.empty(n, H * dk, dtype=bf, device=dev)
        ms = timed(lambda: ops.grouped_linear(qh, wk, qf, n, x_group_cols=dim + rot, o_group_cols=dk), flush=flush)
        fl, by = 2.0 * n * H * rank * dim, (H * rank * dim + n * H * (dim + dk)) * 2
        out[f"fold_keys_into_queries_{label}"] = {"ms": round(ms, 4), "frac": max(frac_flops(fl, ms), frac_bytes(by, ms)),
                                                  "bound": "the larger of both fractions"}
        stream = torch.randn(n, width, device=dev)
        wn = torch.ones(width, device=dev)
        a1, a2 = torch.empty(n, width, dtype=bf, device=dev), torch.empty(n, width, dtype=bf, device=dev)
        ms = timed(lambda: ops.layernorm(stream, wn, 1e-5, a1, None, wn, a2), flush=flush)
        tms = timed(lambda: ops.rmsnorm(stream, wn, 1e-5, a1), flush=flush)
        put(f"norm_{label}", ms, frac_bytes(n * width * 8, ms), tms, frac_bytes(n * width * 6, tms), "copy bandwidth")
        zl = torch.randn(n, E, device=dev)
        wts = torch.empty(n, top, dtype=torch.float32, device=dev)
        ms = timed(lambda: (ops.route(zl, None, z["groups"], z["keep"], top, 1.0, chosen, wts),
                            ops.group_rows(chosen, E, lists[0], lists[1:3], order, place)), flush=flush)
        out[f"route_and_group_{label}"] = {"ms": round(ms, 4), "bound": "latency (two small kernels)"}
        del cache, kc, vc, w1, w2, wd1, wd2
        torch.cuda.empty_cache()
    return out


def compare_nuderax(args, pk):
    import torch
    from bitwise_b200 import Model
    z = NUDERAX_SIZES[args.size]
    line = {"metric": f"Nuderax beside Llama at equal size ({args.size}): prefill of 2,048 tokens and decode at batch "
                      f"{args.batch}, {args.ctx or 2048:,}-token contexts", "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
            "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary", "size": z,
            "peaks": "of " + pk["source"], "l2": "whole models: weights and cache exceed L2; kernels alone: L2 flushed "
            "before every repetition"}
    ctx = args.ctx or 2048
    for name, cfg in (("nuderax", nuderax_config(z)), ("llama_twin", llama_twin(z))):
        model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", fast=True)
        with ClockSampler() as clocks:
            ms, launches = run_decode(model, args.batch, ctx, args.steps, max(3, args.warmup), args.page)
        pms = run_prefill(model, 2048, reps=5, warmup=3, page=args.page)
        line[name] = {"decode_tok_s": round(args.batch / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                      "prefill_tok_s": round(2048 / (pms / 1e3), 1), "prefill_ms": round(pms, 3),
                      "weight_bytes": model.weight_bytes, "gpu_launches": launches, "clocks": clocks.summary()}
        del model
        torch.cuda.empty_cache()
    line["kernels"] = kernel_table(z, pk, args.page)
    return line


# ---- the Favudra design beside Llama at equal size (--compare favudra) -------------------------
FAVUDRA_SIZES = {
    # width, layers, heads, kv_heads, dim = vdim, ff, window, taps, recurrence heads x (dim, vdim), decay rank, vocab
    "small": dict(width=1024, layers=4, heads=8, kv_heads=2, dim=128, ff=2816, window=512, taps=4, rot_dims=64,
                  gla_heads=8, gla_dim=64, gla_vdim=128, decay_rank=32, vocab=32768),
    "medium": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=128, ff=5632, window=1024, taps=4, rot_dims=64,
                   gla_heads=16, gla_dim=128, gla_vdim=128, decay_rank=64, vocab=32768),
}


def favudra_config(z):
    """Layers in the order recurrence, attention, window attention, attention on the second layer's
    keys and values, and so on; every layer with a feed-forward."""
    from bitwise_b200.config import FavudraConfig, FavudraLayerConfig, FavudraMixerConfig
    layers = []
    for i in range(z["layers"]):
        kind = i % 4
        if kind == 0:
            m = FavudraMixerConfig("gla", z["gla_heads"], z["gla_dim"], z["gla_vdim"], tau=16.0, decay_rank=z["decay_rank"])
        elif kind == 2:
            m = FavudraMixerConfig("attention_2", z["heads"], z["dim"], z["dim"], kv_heads=z["kv_heads"],
                                   scale=z["dim"] ** -0.5, window=z["window"])
        else:
            m = FavudraMixerConfig("attention", z["heads"], z["dim"], z["dim"], kv_heads=z["kv_heads"], scale=z["dim"] ** -0.5,
                                   conv=z["taps"], rot_base=1e6, rot_dims=z["rot_dims"], softcap=30.0,
                                   kv_from=i - 2 if kind == 3 else None)
        layers.append(FavudraLayerConfig(m, z["ff"]))
    return FavudraConfig(vocab=z["vocab"], width=z["width"], eps=1e-5, embedding_scale=z["width"] ** 0.5, logit_scale=0.25,
                         layers=tuple(layers))


def favudra_twin(z):
    """Llama with the same width, layers, heads, key/value heads, head size, feed-forward and vocabulary."""
    from bitwise_b200 import LlamaConfig
    return LlamaConfig(vocab_size=z["vocab"], hidden_size=z["width"], num_hidden_layers=z["layers"],
                       num_attention_heads=z["heads"], num_key_value_heads=z["kv_heads"], head_dim=z["dim"],
                       intermediate_size=z["ff"], rope_theta=1e6, rms_norm_eps=1e-5, tie_word_embeddings=False,
                       max_position_embeddings=8192)


def favudra_kernel_table(z, pk, page=16):
    """Every new kernel alone at the size's shapes beside the like kernel of the Llama twin:
    milliseconds and the fraction of its roofline (measured copy bandwidth or bf16 peak)."""
    import torch
    from bitwise_b200.kernels.ops import get_ops
    from bitwise_b200.parts.rope import RotaryEncoding
    from bitwise_b200.parts.scored_attention import SEQUENCE_TILE, distance_slopes
    ops = get_ops("bfloat16")
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, G, hd, width, win, taps = z["heads"], z["kv_heads"], z["dim"], z["width"], z["window"], z["taps"]
    gh, gd, gv = z["gla_heads"], z["gla_dim"], z["gla_vdim"]
    out = {}

    def frac_flops(flops, ms):
        return round(flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"], 4)

    def frac_bytes(nbytes, ms):
        return round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    def put(name, ms, frac, twin_ms, twin_frac, bound):
        out[name] = {"ms": round(ms, 4), "frac": frac, "twin_ms": round(twin_ms, 4), "twin_frac": twin_frac, "bound": bound,
                     "gap_ratio": round(twin_frac / frac, 2) if frac else None}

    cos, sin = RotaryEncoding(z["rot_dims"], 1e6, positions=2048).rotary_tables(dev)
    cos_t, sin_t = RotaryEncoding(hd, 1e6, positions=2048).rotary_tables(dev)
    slopes = torch.tensor(distance_slopes(H), dtype=torch.float32, device=dev)
    for label, seqs in (("prefill_2048", [(0, 2048)]), ("decode_b8_ctx2048", [(2047, 1)] * 8)):
        keys = max(p0 + c for p0, c in seqs)
        blocks = (keys + page - 1) // page
        nseq = len(seqs)
        table = torch.arange(nseq * blocks, dtype=torch.int32, device=dev).reshape(nseq, blocks)
        heights = set(ops.scored_attention_tile_heights(H // G, hd, hd)) | set(ops.attention_tile_heights(H, G, hd)) | {SEQUENCE_TILE}
        b = KernelBatch(seqs, sorted(heights), dev)
        b.seq_slot = torch.arange(nseq, dtype=torch.int32, device=dev)
        n = b.n
        prefill = n > nseq
        pairs = sum(c * p0 + c * (c + 1) // 2 for p0, c in seqs)
        wpairs = sum(sum(min(p + 1, win) for p in range(p0, p0 + c)) for p0, c in seqs)
        kc = torch.randn(nseq * blocks + 1, G, page, hd, device=dev).to(bf)
        vc = torch.randn(nseq * blocks + 1, G, page, hd, device=dev).to(bf)
        q = torch.randn(n, H * hd, device=dev).to(bf)
        o = torch.empty(n, H * hd, dtype=bf, device=dev)
        qkv = torch.randn(n, (H + 2 * G) * hd, device=dev).to(bf)
        twin = lambda w: timed_device(lambda: ops.attention(qkv, kc, vc, table, b.row_seq, b.pos, o, H, G, hd, w, b.max_keys,
                                                     hd ** -0.5, batch=b), flush=flush)
        ms = timed_device(lambda: ops.scored_attention(q, kc, vc, table, o, H, G, hd, hd, hd ** -0.5, 30.0, True, None, 0, b), flush=flush)
        tms = twin(0)
        ms2 = timed_device(lambda: ops.scored_attention(q, kc, None, table, o, H, G, hd, hd, hd ** -0.5, 0.0, False, slopes, win, b),
                    flush=flush)
        tms2 = twin(win)
        if prefill:
            put(f"attention_{label}", ms, frac_flops(4.0 * H * hd * pairs, ms), tms, frac_flops(4.0 * H * hd * pairs, tms), "bf16 peak")
            put(f"window_attention_{label}", ms2, frac_flops(4.0 * H * hd * wpairs, ms2), tms2,
                frac_flops(4.0 * H * hd * wpairs, tms2), "bf16 peak")
        else:
            put(f"attention_{label}", ms, frac_bytes(nseq * keys * 2 * G * hd * 2, ms), tms,
                frac_bytes(nseq * keys * 2 * G * hd * 2, tms), "copy bandwidth")
            put(f"window_attention_{label}", ms2, frac_bytes(nseq * min(keys, win) * G * hd * 2, ms2), tms2,
                frac_bytes(nseq * min(keys, win) * 2 * G * hd * 2, tms2), "copy bandwidth")
        # convolution, norm, rotation and the way into the pages, beside the twin's rotation and store
        cols = (H + 2 * G) * hd
        u = torch.randn(n, cols, device=dev)
        cw = torch.randn(cols, taps, device=dev)
        st = torch.zeros(nseq + 1, taps - 1, cols, device=dev)
        nw = torch.ones(hd, device=dev)
        cwt = cw.t().contiguous()
        ms = timed_device(lambda: (ops.qkv_prepare(u, cw, st, nw, nw, 1e-5, cos, sin, b, table, kc, vc, q, H, G, hd, hd, conv_wt=cwt),
                            ops.conv_state_update(u, st, b, taps, b.query_tiles(SEQUENCE_TILE))), flush=flush)
        tms = timed_device(lambda: ops.rope_cache(qkv, b.pos, b.row_seq, cos_t, sin_t, table, kc, vc, H, G, hd), flush=flush)
        put(f"conv_norm_rotate_store_{label}", ms, frac_bytes(n * cols * 6, ms), tms, frac_bytes(n * cols * 4, tms), "copy bandwidth")
        # the norm after a sublayer beside the twin's norm
        d = torch.randn(n, width, device=dev)
        stream = torch.randn(n, width, device=dev)
        wn = torch.ones(width, device=dev)
        a1 = torch.empty(n, width, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.rmsnorm_residual(d, wn, 1e-5, stream), flush=flush)
        tms = timed_device(lambda: ops.rmsnorm(stream, wn, 1e-5, a1), flush=flush)
        put(f"norm_after_sublayer_{label}", ms, frac_bytes(n * width * 12, ms), tms, frac_bytes(n * width * 6, tms), "copy bandwidth")
        # the recurrence: no like kernel in the twin; per token and head 4 dim vdim operations on the
        # CUDA cores, and in a decode step the state read and written once
        uu = torch.randn(n, 2 * gh * (gd + gv), device=dev)
        zz = torch.randn(n, gh * gd, device=dev)
        state = torch.zeros(nseq + 1, gh, gd, gv, device=dev)
        og = torch.empty(n, gh * gv, dtype=bf, device=dev)
        gb, gw, o32 = torch.zeros(gh * gd, device=dev), torch.ones(gv, device=dev), torch.empty(n, gh * gv, device=dev)
        ms = timed_device(lambda: ops.gla_scan(uu, zz, gb, 16.0, state, gw, 1e-5, og, gh, gd, gv, gd ** -0.5, b,
                                               b.query_tiles(SEQUENCE_TILE), scratch=o32), flush=flush)
        if prefill:
            out[f"recurrence_{label}"] = {"ms": round(ms, 4), "frac": round(4.0 * n * gh * gd * gv / (ms / 1e3) / 1e12 /
                                                                             pk.get("fp32_tflops", 74.0), 4),
                                          "bound": "float32 on the CUDA cores; a sequence's tokens are walked one after the other"}
        else:
            out[f"recurrence_{label}"] = {"ms": round(ms, 4), "frac": frac_bytes(nseq * gh * gd * gv * 8, ms), "bound": "copy bandwidth"}
        del kc, vc
        torch.cuda.empty_cache()
    return out


def compare_favudra(args, pk):
    import torch
    from bitwise_b200 import Model
    z = FAVUDRA_SIZES[args.size]
    line = {"metric": f"Favudra beside Llama at equal size ({args.size}): prefill of 2,048 tokens and decode at batch "
                      f"{args.batch}, {args.ctx or 2048:,}-token contexts", "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
            "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary", "size": z,
            "peaks": "of " + pk["source"], "l2": "whole models: weights and cache exceed L2; kernels alone: L2 flushed "
            "before every repetition"}
    ctx = args.ctx or 2048
    for name, cfg in (("favudra", favudra_config(z)), ("llama_twin", favudra_twin(z))):
        model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", fast=True)
        with ClockSampler() as clocks:
            ms, launches = run_decode(model, args.batch, ctx, args.steps, max(3, args.warmup), args.page)
        pms = run_prefill(model, 2048, reps=5, warmup=3, page=args.page)
        line[name] = {"decode_tok_s": round(args.batch / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                      "prefill_tok_s": round(2048 / (pms / 1e3), 1), "prefill_ms": round(pms, 3),
                      "weight_bytes": model.weight_bytes, "gpu_launches": launches, "clocks": clocks.summary()}
        del model
        torch.cuda.empty_cache()
    line["kernels"] = favudra_kernel_table(z, pk, args.page)
    return line


# ---- the Sebavik design beside Favudra at equal size (--compare sebavik) ------------------------
SEBAVIK_SIZES = {
    # width, layers, heads, kv_heads, dim = vdim, dense ff, window with kept first keys, taps, experts x top x ff,
    # second table's buckets, token input's size, vocab
    "small": dict(width=1024, layers=4, heads=8, kv_heads=2, dim=128, ff=2816, window=512, keep_first=4, taps=4,
                  experts=8, top=2, expert_ff=1408, buckets=65521, side_dim=32, vocab=32768),
    "medium": dict(width=2048, layers=4, heads=16, kv_heads=4, dim=128, ff=5632, window=1024, keep_first=16, taps=4,
                   experts=16, top=4, expert_ff=1408, buckets=131071, side_dim=64, vocab=32768),
}


def sebavik_config(z):
    """Layers alternate a dense and a routed feed-forward (the routed one multiplies a token with as many inner
    columns as the dense one: top x expert ff = ff); every layer's attention has the window, the cap, the distance
    term and the sink, and all but the first mix their values with the first layer's."""
    from bitwise_b200.config.sebavik import BigramConfig, SebavikConfig, SebavikLayerConfig, SebavikMixerConfig, SebavikMlpConfig
    layers = []
    for i in range(z["layers"]):
        m = SebavikMixerConfig(heads=z["heads"], kv_heads=z["kv_heads"], dim=z["dim"], vdim=z["dim"], scale=z["dim"] ** -0.5,
                               softcap=30.0, window=z["window"], keep_first=z["keep_first"], v_mix=True)
        mlp = SebavikMlpConfig("dense", z["ff"], 7.0) if i % 2 == 0 else SebavikMlpConfig("moe", z["expert_ff"], None,
                                                                                          z["experts"], z["top"])
        layers.append(SebavikLayerConfig(m, mlp))
    return SebavikConfig(vocab=z["vocab"], width=z["width"], eps=1e-5, residual_mult=0.5, embedding_scale=z["width"] ** 0.5,
                         layers=tuple(layers), bigram=BigramConfig(z["buckets"], 40503, 2971), canon_taps=z["taps"],
                         side_dim=z["side_dim"])


def sebavik_twin(z):
    """Favudra with the same width, layers, heads, key/value heads, head size, feed-forward and vocabulary, its
    layers alternating capped attention with a sink (and the convolution on q, k, v) and window attention."""
    from bitwise_b200.config import FavudraConfig, FavudraLayerConfig, FavudraMixerConfig
    layers = []
    for i in range(z["layers"]):
        if i % 2 == 0:
            m = FavudraMixerConfig("attention", z["heads"], z["dim"], z["dim"], kv_heads=z["kv_heads"], scale=z["dim"] ** -0.5,
                                   conv=z["taps"], rot_base=1e6, rot_dims=64, softcap=30.0)
        else:
            m = FavudraMixerConfig("attention_2", z["heads"], z["dim"], z["dim"], kv_heads=z["kv_heads"],
                                   scale=z["dim"] ** -0.5, window=z["window"])
        layers.append(FavudraLayerConfig(m, z["ff"]))
    return FavudraConfig(vocab=z["vocab"], width=z["width"], eps=1e-5, embedding_scale=z["width"] ** 0.5, logit_scale=0.25,
                         layers=tuple(layers))


def sebavik_kernel_table(z, pk, page=16):
    """Every kernel that the design adds or extends, alone at the size's shapes, beside the like kernel of the twin:
    milliseconds and the fraction of its roofline (measured copy bandwidth or bf16 peak)."""
    import torch
    from bitwise_b200.kernels.ops import get_ops
    from bitwise_b200.parts.rope import RotaryEncoding
    from bitwise_b200.parts.scored_attention import SEQUENCE_TILE, distance_slopes
    ops = get_ops("bfloat16")
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, G, hd, width, win, keep, taps = z["heads"], z["kv_heads"], z["dim"], z["width"], z["window"], z["keep_first"], z["taps"]
    L, sd, vocab = z["layers"], z["side_dim"], z["vocab"]
    out = {}

    def frac_flops(flops, ms):
        return round(flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"], 4)

    def frac_bytes(nbytes, ms):
        return round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    def put(name, ms, frac, twin_ms, twin_frac, bound, twin):
        out[name] = {"ms": round(ms, 4), "frac": frac, "twin_ms": round(twin_ms, 4), "twin_frac": twin_frac, "bound": bound,
                     "twin": twin, "gap_ratio": round(twin_frac / frac, 2) if frac else None}

    cos, sin = RotaryEncoding(64, 1e6, positions=2048).rotary_tables(dev)
    slopes = torch.tensor(distance_slopes(H), dtype=torch.float32, device=dev)
    r1 = torch.full((H,), 0.3, device=dev)
    r2 = torch.full((H,), 0.5, device=dev)
    sinks = torch.zeros(H, device=dev)
    for label, seqs in (("prefill_2048", [(0, 2048)]), ("decode_b8_ctx2048", [(2047, 1)] * 8)):
        keys = max(p0 + c for p0, c in seqs)
        blocks = (keys + page - 1) // page
        nseq = len(seqs)
        table = torch.arange(nseq * blocks, dtype=torch.int32, device=dev).reshape(nseq, blocks)
        heights = set(ops.scored_attention_tile_heights(H // G, hd, hd)) | {SEQUENCE_TILE}
        b = KernelBatch(seqs, sorted(heights), dev)
        b.seq_slot = torch.arange(nseq, dtype=torch.int32, device=dev)
        b.tokens = torch.randint(0, vocab, (b.n,), dtype=torch.int32, device=dev)
        n = b.n
        prefill = n > nseq
        seen = lambda p: min(p + 1, win) + max(0, min(keep, p + 1 - win))
        wpairs = sum(sum(seen(p) for p in range(p0, p0 + c)) for p0, c in seqs)
        kc = torch.randn(nseq * blocks + 1, G, page, hd, device=dev).to(bf)
        vc = torch.randn(nseq * blocks + 1, G, page, hd, device=dev).to(bf)
        q = torch.randn(n, H * hd, device=dev).to(bf)
        o = torch.empty(n, H * hd, dtype=bf, device=dev)
        # window attention with kept first keys, cap, logarithmic distance term and learned sink, beside the twin's
        # window attention with distance slopes (whose values are its keys)
        ms = timed_device(lambda: ops.scored_attention(q, kc, vc, table, o, H, G, hd, hd, hd ** -0.5, 30.0, True, None, win, b,
                                                       dist_a=r1, dist_b=r2, sinks=sinks, keep_first=keep), flush=flush)
        tms = timed_device(lambda: ops.scored_attention(q, kc, None, table, o, H, G, hd, hd, hd ** -0.5, 0.0, False, slopes, win, b),
                           flush=flush)
        if prefill:
            put(f"attention_{label}", ms, frac_flops(4.0 * H * hd * wpairs, ms), tms, frac_flops(4.0 * H * hd * wpairs, tms),
                "bf16 peak", "window attention with slopes")
        else:
            put(f"attention_{label}", ms, frac_bytes(nseq * seen(keys - 1) * 2 * G * hd * 2, ms), tms,
                frac_bytes(nseq * min(keys, win) * G * hd * 2, tms), "copy bandwidth", "window attention with slopes")
        # biases, mixed values and the way into the pages, beside the twin's convolution, norm, rotation and store
        cols = (H + 2 * G) * hd
        u = torch.randn(n, cols, device=dev)
        bias = torch.randn(cols, device=dev)
        first = torch.randn(n, G * hd, device=dev)
        lam = torch.full((1,), 0.3, device=dev)
        cw = torch.randn(cols, taps, device=dev)
        st = torch.zeros(nseq + 1, taps - 1, cols, device=dev)
        nw = torch.ones(hd, device=dev)
        cwt = cw.t().contiguous()
        ms = timed_device(lambda: ops.qkv_prepare(u, None, None, None, None, 1e-5, None, None, b, table, kc, vc, q, H, G, hd, hd,
                                                  bias=bias, vmix_src=first, vmix_lambda=lam), flush=flush)
        tms = timed_device(lambda: (ops.qkv_prepare(u, cw, st, nw, nw, 1e-5, cos, sin, b, table, kc, vc, q, H, G, hd, hd, conv_wt=cwt),
                                    ops.conv_state_update(u, st, b, taps, b.query_tiles(SEQUENCE_TILE))), flush=flush)
        put(f"bias_mix_store_{label}", ms, frac_bytes(n * (cols * 6 + G * hd * 4), ms), tms, frac_bytes(n * cols * 6, tms),
            "copy bandwidth", "convolution, norm, rotation, store")
        # the norm with the convolution over time (and the state's update), beside the twin's norm
        stream = torch.randn(n, width, device=dev)
        wn = torch.ones(width, device=dev)
        taps_t = torch.randn(taps, width, device=dev)
        cst = torch.zeros(nseq + 1, taps - 1, 2 * width, device=dev)
        normed = torch.empty(n, 2 * width, device=dev)
        a1 = torch.empty(n, width, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.norm_conv(stream, wn, 1e-5, taps_t, cst, 0, b, a1, normed, 0), flush=flush)
        tms = timed_device(lambda: ops.rmsnorm(stream, wn, 1e-5, a1), flush=flush)
        put(f"norm_conv_{label}", ms, frac_bytes(n * width * 6, ms), tms, frac_bytes(n * width * 6, tms), "copy bandwidth", "norm")
        ms = timed_device(lambda: ops.conv_state_update(normed, cst, b, taps, b.query_tiles(SEQUENCE_TILE)), flush=flush)
        out[f"conv_state_update_{label}"] = {"ms": round(ms, 4), "bound": "launch: taps - 1 rows per sequence"}
        # the scaled sum of a sublayer's output, and the token input's norm with the depth average, beside the
        # twin's norm after a sublayer
        d = torch.randn(n, width, device=dev)
        scale = torch.ones(width, device=dev)
        history = torch.randn(n, (L + 1) * width, device=dev)
        mix = torch.full((L + 1,), 0.2, device=dev)
        tms = timed_device(lambda: ops.rmsnorm_residual(d, wn, 1e-5, stream), flush=flush)
        ms = timed_device(lambda: ops.scaled_add(stream, scale, d, a1), flush=flush)
        put(f"scaled_sum_{label}", ms, frac_bytes(n * width * 14, ms), tms, frac_bytes(n * width * 12, tms), "copy bandwidth",
            "norm after a sublayer")
        ms = timed_device(lambda: ops.normed_add_mix(stream, d, wn, 1e-5, 0.5, history, L, mix), flush=flush)
        put(f"side_norm_depth_average_{label}", ms, frac_bytes(n * width * (16 + 4 * L), ms), tms, frac_bytes(n * width * 12, tms),
            "copy bandwidth", "norm after a sublayer")
        # the embedding with the second table, beside the twin's embedding
        emb = torch.randn(vocab, width, device=dev).to(bf)
        pair = torch.randn(z["buckets"] + 1, width, device=dev).to(bf)
        last = torch.zeros(nseq + 1, 1, dtype=torch.int32, device=dev)
        ms = timed_device(lambda: (ops.embed_pair(emb, pair, b, last, stream, 2.0, z["buckets"], 40503, 2971),
                                   ops.last_token_update(b, last, b.query_tiles(SEQUENCE_TILE))), flush=flush)
        tms = timed_device(lambda: ops.embed_rows(emb, b.tokens, stream, scale=2.0), flush=flush)
        put(f"embedding_{label}", ms, frac_bytes(n * width * 8, ms), tms, frac_bytes(n * width * 6, tms), "copy bandwidth", "embedding")
        # the token input's gate
        t = torch.randn(n, sd, device=dev)
        side = torch.randn(vocab, L * sd, device=dev).to(bf)
        g = torch.empty(n, sd, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.token_gate(t, side, sd, b.tokens, g), flush=flush)
        out[f"token_gate_{label}"] = {"ms": round(ms, 4), "frac": frac_bytes(n * sd * 8, ms), "bound": "copy bandwidth (launch at these sizes)"}
        # the router: the softmax over the chosen logits beside the sigmoid scores of the routed design
        E, top = z["experts"], z["top"]
        logits = torch.randn(n, E, device=dev)
        chosen = torch.empty(n, top, dtype=torch.int32, device=dev)
        weights = torch.empty(n, top, device=dev)
        ms = timed_device(lambda: ops.route(logits, None, 1, 1, top, 1.0, chosen, weights, softmax_top=True), flush=flush)
        tms = timed_device(lambda: ops.route(logits, None, 1, 1, top, 1.0, chosen, weights), flush=flush)
        put(f"route_{label}", ms, frac_bytes(n * (E * 4 + top * 8), ms), tms, frac_bytes(n * (E * 4 + top * 8), tms),
            "copy bandwidth (launch at these sizes)", "sigmoid scores")
        del kc, vc, emb, pair, side, history
        torch.cuda.empty_cache()
    return out


def compare_sebavik(args, pk):
    import torch
    from bitwise_b200 import Model
    z = SEBAVIK_SIZES[args.size]
    ctx = args.ctx or 2048
    line = {"metric": f"Sebavik beside Favudra at equal size ({args.size}): prefill of 2,048 tokens and decode at batch "
                      f"{args.batch}, {ctx:,}-token contexts", "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
            "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary", "size": z,
            "peaks": "of " + pk["source"], "l2": "whole models: weights and cache exceed L2; kernels alone: L2 flushed "
            "before every repetition"}
    for name, cfg in (("sebavik", sebavik_config(z)), ("favudra_twin", sebavik_twin(z))):
        model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", fast=True)
        with ClockSampler() as clocks:
            ms, launches = run_decode(model, args.batch, ctx, args.steps, max(3, args.warmup), args.page)
        pms = run_prefill(model, 2048, reps=5, warmup=3, page=args.page)
        line[name] = {"decode_tok_s": round(args.batch / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                      "prefill_tok_s": round(2048 / (pms / 1e3), 1), "prefill_ms": round(pms, 3),
                      "weight_bytes": model.weight_bytes, "gpu_launches": launches, "clocks": clocks.summary()}
        del model
        torch.cuda.empty_cache()
    line["kernels"] = sebavik_kernel_table(z, pk, args.page)
    return line

# ---- the Kezuvik design beside Favudra at equal size (--compare kezuvik) ------------------------
KEZUVIK_SIZES = {
    # width, layers, latent layers: heads x (dim + rot_dim), value size, latents of keys/values and of queries;
    # window layers: heads on kv_heads of dim, window, taps; ff, vocab
    "small": dict(width=1024, layers=4, heads=8, dim=64, rot_dim=32, vdim=64, kv_rank=256, q_rank=384,
                  w_heads=8, w_kv_heads=2, w_dim=128, window=512, taps=4, ff=2816, vocab=32768),
    "medium": dict(width=2048, layers=4, heads=16, dim=128, rot_dim=64, vdim=128, kv_rank=512, q_rank=768,
                   w_heads=16, w_kv_heads=4, w_dim=128, window=1024, taps=4, ff=5632, vocab=32768),
}


def kezuvik_config(z):
    """Layers in the order latent attention, window attention, latent attention of the second kind (rescaled rotary
    frequencies, sinks, a gate per head), window attention, and so on; every layer with a feed-forward."""
    from bitwise_b200.config import KezuvikConfig, KezuvikLayerConfig, KezuvikMixerConfig, RotScalingConfig
    layers = []
    for i in range(z["layers"]):
        kind = i % 4
        if kind in (1, 3):
            m = KezuvikMixerConfig("attention", z["w_heads"], z["w_dim"], z["w_dim"], z["w_dim"] ** -0.5,
                                   kv_heads=z["w_kv_heads"], conv=z["taps"], window=z["window"])
        else:
            m = KezuvikMixerConfig("latent_attention_2" if kind == 2 else "latent_attention", z["heads"], z["dim"], z["vdim"],
                                   (z["dim"] + z["rot_dim"]) ** -0.5, rot_dim=z["rot_dim"], kv_rank=z["kv_rank"],
                                   q_rank=z["q_rank"], rot_base=1e6, rot_dims=z["rot_dim"],
                                   rot_scaling=RotScalingConfig(4.0, 4096.0, 32.0, 1.0) if kind == 2 else None)
        layers.append(KezuvikLayerConfig(m, z["ff"]))
    return KezuvikConfig(vocab=z["vocab"], width=z["width"], eps=1e-5, layers=tuple(layers), residual_mult=0.7,
                         logit_softcap=30.0)


def kezuvik_twin(z):
    """Favudra with the same width, layers, feed-forward and vocabulary and the window layers' heads, key/value heads
    and head size: full attention (convolution, norm per head, rotation, cap, sink) where Kezuvik has latent attention,
    window attention where it has window attention."""
    from bitwise_b200.config import FavudraConfig, FavudraLayerConfig, FavudraMixerConfig
    H, G, hd = z["w_heads"], z["w_kv_heads"], z["w_dim"]
    layers = []
    for i in range(z["layers"]):
        if i % 2:
            m = FavudraMixerConfig("attention_2", H, hd, hd, kv_heads=G, scale=hd ** -0.5, window=z["window"])
        else:
            m = FavudraMixerConfig("attention", H, hd, hd, kv_heads=G, scale=hd ** -0.5, conv=z["taps"], rot_base=1e6,
                                   rot_dims=64, softcap=30.0)
        layers.append(FavudraLayerConfig(m, z["ff"]))
    return FavudraConfig(vocab=z["vocab"], width=z["width"], eps=1e-5, embedding_scale=z["width"] ** 0.5, logit_scale=0.25,
                         layers=tuple(layers))


def kezuvik_kernel_table(z, pk, page=16):
    """Every kernel that the design added or changed, alone at the size's shapes, beside the like kernel of an
    earlier design: milliseconds and the fraction of its roofline (measured copy bandwidth or bf16 peak)."""
    import torch
    from bitwise_b200.kernels.ops import get_ops
    from bitwise_b200.parts.rope import HalfRotaryEncoding, RampScaling, RotaryEncoding
    from bitwise_b200.parts.scored_attention import SEQUENCE_TILE, distance_slopes
    ops = get_ops("bfloat16")
    dev, bf = "cuda:0", torch.bfloat16
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    H, rank, rot, dim, vdim, width = z["heads"], z["kv_rank"], z["rot_dim"], z["dim"], z["vdim"], z["width"]
    WH, WG, hd, win, taps, ff = z["w_heads"], z["w_kv_heads"], z["w_dim"], z["window"], z["taps"], z["ff"]
    dk = rank + rot
    out = {}

    def frac_flops(flops, ms):
        return round(flops / (ms / 1e3) / 1e12 / pk["bf16_tflops"], 4)

    def frac_bytes(nbytes, ms):
        return round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)

    def put(name, ms, frac, twin_ms, twin_frac, bound, twin):
        out[name] = {"ms": round(ms, 4), "frac": frac, "twin_ms": round(twin_ms, 4), "twin_frac": twin_frac, "bound": bound,
                     "twin": twin, "gap_ratio": round(twin_frac / frac, 2) if frac else None}

    cos_h, sin_h = HalfRotaryEncoding(rot, 1e6, RampScaling(4.0, 4096.0, 32.0, 1.0), positions=2048).rotary_tables(dev)
    cos_p, sin_p = RotaryEncoding(rot, 1e6, positions=2048).rotary_tables(dev)
    cos_f, sin_f = RotaryEncoding(64, 1e6, positions=2048).rotary_tables(dev)
    slopes = torch.tensor(distance_slopes(WH), dtype=torch.float32, device=dev)
    sinks = torch.zeros(H, dtype=torch.float32, device=dev)
    for label, seqs in (("prefill_2048", [(0, 2048)]), ("decode_b8_ctx2048", [(2047, 1)] * 8)):
        keys = max(p0 + c for p0, c in seqs)
        blocks = (keys + page - 1) // page
        nseq = len(seqs)
        table = torch.arange(nseq * blocks, dtype=torch.int32, device=dev).reshape(nseq, blocks)
        heights = set(ops.latent_attention_tile_heights(H, rank, rot)) | set(ops.scored_attention_tile_heights(WH // WG, hd, hd)) | {SEQUENCE_TILE}
        b = KernelBatch(seqs, sorted(heights), dev)
        b.seq_slot = torch.arange(nseq, dtype=torch.int32, device=dev)
        n = b.n
        prefill = n > nseq
        pairs = sum(c * p0 + c * (c + 1) // 2 for p0, c in seqs)
        wpairs = sum(sum(min(p + 1, win) for p in range(p0, p0 + c)) for p0, c in seqs)
        # latent attention with a sink per head beside the same attention without (the Nuderax design's)
        cache = torch.randn(nseq * blocks + 1, page, dk, device=dev).to(bf)
        q = torch.randn(n, H * dk, device=dev).to(bf)
        o = torch.empty(n, H * rank, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.latent_attention(q, cache, table, o, H, rank, rot, dk ** -0.5, b, sinks=sinks), flush=flush)
        tms = timed_device(lambda: ops.latent_attention(q, cache, table, o, H, rank, rot, dk ** -0.5, b), flush=flush)
        if prefill:
            fl = 2.0 * H * (dk + rank) * pairs
            put(f"latent_attention_sink_{label}", ms, frac_flops(fl, ms), tms, frac_flops(fl, tms), "bf16 peak", "latent attention")
        else:
            by = nseq * keys * dk * 2
            put(f"latent_attention_sink_{label}", ms, frac_bytes(by, ms), tms, frac_bytes(by, tms), "copy bandwidth", "latent attention")
        # the latent and the rotated parts on their way into the pages and into the folded queries: half layout beside pairs
        d = torch.randn(n, dk, device=dev)
        wn = torch.ones(rank, device=dev)
        qh = torch.randn(n, H * (dim + rot), device=dev).to(bf)
        qf = torch.empty(n, H * dk, dtype=bf, device=dev)
        run = lambda c, s_, half: (ops.latent_store(d, wn, 1e-5, b.pos, b.row_seq, c, s_, table, cache, rank, rot, half_layout=half),
                                   ops.rotate_heads(qh, H, dim + rot, dim, rot, qf, dk, rank, b.pos, c, s_, half_layout=half))
        ms = timed_device(lambda: run(cos_h, sin_h, True), flush=flush)
        tms = timed_device(lambda: run(cos_p, sin_p, False), flush=flush)
        by = n * (dk * 6 + H * rot * 4)
        put(f"store_and_rotate_{label}", ms, frac_bytes(by, ms), tms, frac_bytes(by, tms), "copy bandwidth", "the same kernels, pairs (2i, 2i + 1)")
        # window attention (no cap, no sink, values of their own) beside Favudra's window attention (slopes, values = keys)
        kc = torch.randn(nseq * blocks + 1, WG, page, hd, device=dev).to(bf)
        vc = torch.randn(nseq * blocks + 1, WG, page, hd, device=dev).to(bf)
        wq = torch.randn(n, WH * hd, device=dev).to(bf)
        wo = torch.empty(n, WH * hd, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.scored_attention(wq, kc, vc, table, wo, WH, WG, hd, hd, hd ** -0.5, 0.0, False, None, win, b), flush=flush)
        tms = timed_device(lambda: ops.scored_attention(wq, kc, None, table, wo, WH, WG, hd, hd, hd ** -0.5, 0.0, False, slopes, win, b),
                           flush=flush)
        if prefill:
            fl = 4.0 * WH * hd * wpairs
            put(f"window_attention_{label}", ms, frac_flops(fl, ms), tms, frac_flops(fl, tms), "bf16 peak", "window attention with slopes")
        else:
            by = nseq * min(keys, win) * WG * hd * 2
            put(f"window_attention_{label}", ms, frac_bytes(2 * by, ms), tms, frac_bytes(by, tms), "copy bandwidth",
                "window attention with slopes (keys only)")
        # biases, convolution, unit norm and store beside Favudra's convolution, weighted norm, rotation and store
        cols = (WH + 2 * WG) * hd
        u = torch.randn(n, cols, device=dev)
        cw = torch.randn(cols, taps, device=dev)
        cwt = cw.t().contiguous()
        st = torch.zeros(nseq + 1, taps - 1, cols, device=dev)
        nw = torch.ones(hd, device=dev)
        bias = torch.randn(cols, device=dev)
        ms = timed_device(lambda: (ops.qkv_prepare(u, cw, st, nw, nw, 1e-5, None, None, b, table, kc, vc, wq, WH, WG, hd, hd, conv_wt=cwt, bias=bias),
                                   ops.conv_state_update(u, st, b, taps, b.query_tiles(SEQUENCE_TILE))), flush=flush)
        tms = timed_device(lambda: (ops.qkv_prepare(u, cw, st, nw, nw, 1e-5, cos_f, sin_f, b, table, kc, vc, wq, WH, WG, hd, hd, conv_wt=cwt),
                                    ops.conv_state_update(u, st, b, taps, b.query_tiles(SEQUENCE_TILE))), flush=flush)
        put(f"bias_conv_norm_store_{label}", ms, frac_bytes(n * cols * 6, ms), tms, frac_bytes(n * cols * 6, tms), "copy bandwidth",
            "convolution, norm, rotation, store")
        # the layer norm after a sublayer (with the next sublayer's norm) beside the root-mean-square one
        dd = torch.randn(n, width, device=dev)
        stream = torch.randn(n, width, device=dev)
        ww = torch.ones(width, device=dev)
        a1 = torch.empty(n, width, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.layernorm_residual(dd, ww, 1e-5, stream, next_weight=ww, next_eps=1e-5, next_out=a1), flush=flush)
        tms = timed_device(lambda: ops.rmsnorm_residual(dd, ww, 1e-5, stream, next_weight=ww, next_eps=1e-5, next_out=a1), flush=flush)
        put(f"norm_after_sublayer_{label}", ms, frac_bytes(n * width * 14, ms), tms, frac_bytes(n * width * 14, tms), "copy bandwidth",
            "root-mean-square norm after a sublayer")
        # the output gate beside the stand-alone gated step (both read two numbers and write one per output)
        hv = torch.randn(n, H * vdim, device=dev).to(bf)
        gl = torch.randn(n, H * vdim, device=dev)
        gh = torch.randn(n, H, device=dev)
        gu = torch.randn(n, 2 * H * vdim, device=dev).to(bf)
        ms = timed_device(lambda: ops.sigmoid_gate(hv, gl, 1), flush=flush)
        ms_h = timed_device(lambda: ops.sigmoid_gate(hv, gh, vdim), flush=flush)
        tms = timed_device(lambda: ops.swiglu(gu, hv), flush=flush)
        put(f"gate_per_entry_{label}", ms, frac_bytes(n * H * vdim * 8, ms), tms, frac_bytes(n * H * vdim * 6, tms), "copy bandwidth",
            "stand-alone SwiGLU")
        put(f"gate_per_head_{label}", ms_h, frac_bytes(n * H * vdim * 4, ms_h), tms, frac_bytes(n * H * vdim * 6, tms), "copy bandwidth",
            "stand-alone SwiGLU")
        # the gate/up product with the GELU form in its epilogue beside the same product with SiLU
        x = torch.randn(n, width, device=dev).to(bf)
        wgu = (torch.randn(2 * ff, width, device=dev) * 0.02).to(bf)
        hh = torch.empty(n, ff, dtype=bf, device=dev)
        ms = timed_device(lambda: ops.linear_swiglu(x, wgu, hh, activation="gelu_tanh"), flush=flush)
        tms = timed_device(lambda: ops.linear_swiglu(x, wgu, hh), flush=flush)
        if prefill:
            fl = 2.0 * n * 2 * ff * width
            put(f"gate_up_gelu_{label}", ms, frac_flops(fl, ms), tms, frac_flops(fl, tms), "bf16 peak", "gate/up product with SiLU")
        else:
            by = 2 * ff * width * 2
            put(f"gate_up_gelu_{label}", ms, frac_bytes(by, ms), tms, frac_bytes(by, tms), "copy bandwidth", "gate/up product with SiLU")
        # the cap on the logits of the step's wanted rows (no like kernel)
        rows = 8 if not prefill else 1
        lg = torch.randn(rows, z["vocab"], device=dev)
        ms = timed_device(lambda: ops.softcap_rows(lg, 30.0), flush=flush)
        out[f"logit_cap_{label}"] = {"ms": round(ms, 4), "bound": "latency (one small kernel)"}
        del cache, kc, vc, wgu
        torch.cuda.empty_cache()
    return out


def compare_kezuvik(args, pk):
    import torch
    from bitwise_b200 import Model
    z = KEZUVIK_SIZES[args.size]
    line = {"metric": f"Kezuvik beside Favudra at equal size ({args.size}): prefill of 2,048 tokens and decode at batch "
                      f"{args.batch}, {args.ctx or 2048:,}-token contexts", "unit": "tokens/s", "n_gpus": 1, "dtype": "bf16",
            "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary", "size": z,
            "peaks": "of " + pk["source"], "l2": "whole models: weights and cache exceed L2; kernels alone: L2 flushed "
            "before every repetition"}
    ctx = args.ctx or 2048
    for name, cfg in (("kezuvik", kezuvik_config(z)), ("favudra_twin", kezuvik_twin(z))):
        model = Model.random(cfg, seed=0, dtype="bfloat16", device="cuda:0", fast=True)
        with ClockSampler() as clocks:
            ms, launches = run_decode(model, args.batch, ctx, args.steps, max(3, args.warmup), args.page)
        pms = run_prefill(model, 2048, reps=5, warmup=3, page=args.page)
        line[name] = {"decode_tok_s": round(args.batch / (ms / 1e3), 1), "decode_ms_per_step": round(ms, 4),
                      "prefill_tok_s": round(2048 / (pms / 1e3), 1), "prefill_ms": round(pms, 3),
                      "weight_bytes": model.weight_bytes, "gpu_launches": launches, "clocks": clocks.summary()}
        del model
        torch.cuda.empty_cache()
    line["kernels"] = kezuvik_kernel_table(z, pk, args.page)
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="smollm2-1.7b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=0, help="layers to run (default: all of the shape's)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=0, help="tokens in each request's cache (default: the shape's)")
    ap.add_argument("--workload", default="decode", choices=["decode", "serve"],
                    help="serve: 64 requests with prompts of 16..1024 and outputs of 16..256 tokens through the "
                         "engine's scheduler under a 512-token budget")
    ap.add_argument("--skip-fp32", action="store_true", help="leave out the float32 figures")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--skip-points", action="store_true", help="only the headline decode (for profiling runs)")
    ap.add_argument("--skip-prefill", action="store_true")
    ap.add_argument("--compare", default="", choices=["", "nuderax", "favudra", "sebavik", "kezuvik"],
                    help="instead of the headline: this design beside its closest earlier architecture at equal size")
    ap.add_argument("--size", default="small", choices=sorted(set(NUDERAX_SIZES) | set(FAVUDRA_SIZES) | set(SEBAVIK_SIZES) | set(KEZUVIK_SIZES)),
                    help="layer sizes for --compare")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        print(json.dumps(reference_arm(args)))
        return 0
    warmup = max(3, args.warmup)

    import torch
    from bitwise_b200 import Model
    pk = peaks()
    if args.compare == "nuderax":
        print(json.dumps(compare_nuderax(args, pk)))
        return 0
    if args.compare == "favudra":
        print(json.dumps(compare_favudra(args, pk)))
        return 0
    if args.compare == "kezuvik":
        print(json.dumps(compare_kezuvik(args, pk)))
        return 0
    if args.compare == "sebavik":
        print(json.dumps(compare_sebavik(args, pk)))
        return 0
    title, full_layers, _, shape_ctx = SHAPES[args.shape]
    args.layers = args.layers or full_layers
    args.ctx = args.ctx or shape_ctx
    cfg = model_config(args.shape, args.layers)
    model = Model.random(cfg, seed=0, dtype=args.dtype, device="cuda:0", fast=True)
    elt = 2 if args.dtype == "bfloat16" else 4
    if args.workload == "serve":
        print(json.dumps(run_serve(model, title, args, pk)))
        return 0

    with ClockSampler() as clocks:
        ms, launches = run_decode(model, args.batch, args.ctx, args.steps, warmup, args.page)
    value = args.batch / (ms / 1e3)
    bytes_step = decode_bytes(cfg, args.batch, args.ctx, elt)
    achieved = bytes_step / (ms / 1e3) / 1e9

    line = {
        "metric": f"decode tok/s at batch {args.batch}, {args.ctx:,}-token context ({title})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": baseline_ratio(args, value), "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary",
        "impl": "ours",
        "config": {"model": title, "layers": full_layers, "layers_run": args.layers,
                   "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads,
                   "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
                   "tied_embeddings": cfg.tie_word_embeddings, "global_batch": args.batch, "seq_len": args.ctx,
                   "page_size": args.page, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights + cache read per step exceed 126 MB)",
                   "peaks": "of " + pk["source"], "baseline": BASELINE_NOTE},
        "clocks": clocks.summary(),
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": bytes_step},
    }
    if not args.skip_prefill:
        pms = run_prefill(model, 2048, reps=5, warmup=3, page=args.page)
        fl = prefill_flops(cfg, 2048)
        peak_tf = pk["bf16_tflops"] if args.dtype == "bfloat16" else fp32_simt_tflops()
        line["prefill"] = {"value": round(2048 / (pms / 1e3), 1), "tokens": 2048, "ms": round(pms, 3),
                           "frac": round(fl / (pms / 1e3) / 1e12 / peak_tf, 4), "flops": fl}
        if args.dtype != "bfloat16":
            line["prefill"]["peak"] = "float32 on the CUDA cores, %.1f TFLOP/s nominal" % peak_tf
    if not args.skip_points:
        pts = {}
        for b in (1, 64):
            pm, _ = run_decode(model, b, args.ctx, max(10, args.steps // 2), 3, args.page)
            pts[f"decode_b{b}"] = round(b / (pm / 1e3), 1)
            pts[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, args.ctx, elt) / (pm / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        line["points"] = pts
        e, h2d, d2h = run_e2e(model, args.batch, args.ctx, args.steps, warmup, args.page, fingerprint=True)
        e_plain, _, _ = run_e2e(model, args.batch, args.ctx, args.steps, warmup, args.page, fingerprint=False)
        line["e2e"] = {"value": round(e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "settings": "Engine defaults (fingerprint_logits on, a step ahead of the reads)",
                       "value_without_fingerprint": round(e_plain, 1)}
    if not args.skip_fp32 and args.dtype == "bfloat16" and not args.skip_points:
        # the true 32-bit path of the same shape (no reduced-precision matrix mode anywhere)
        del model
        torch.cuda.empty_cache()
        m32 = Model.random(cfg, seed=0, dtype="float32", device="cuda:0", fast=True)
        fm, _ = run_decode(m32, args.batch, args.ctx, max(5, args.steps // 5), 3, args.page)
        f32 = {"decode_b%d" % args.batch: round(args.batch / (fm / 1e3), 1), "ms_per_step": round(fm, 3),
               "decode_hbm_frac": round(decode_bytes(cfg, args.batch, args.ctx, 4) / (fm / 1e3) / 1e9 / pk["hbm_gbs"], 4)}
        if not args.skip_prefill:
            fp = run_prefill(m32, 2048, reps=3, warmup=3, page=args.page)
            f32["prefill"] = round(2048 / (fp / 1e3), 1)
            f32["prefill_ms"] = round(fp, 2)
            # against the float32 peak of the CUDA cores (no tensor core on this path)
            f32["prefill_frac"] = round(prefill_flops(cfg, 2048) / (fp / 1e3) / 1e12 / fp32_simt_tflops(), 4)
        line["fp32"] = f32
    print(json.dumps(line))
    return 0


BASELINE_NOTE = ("vs_baseline divides by BASELINE.md's figure for the same shape, batch and context: the reference's "
                 "Runner::forward on this image's CPU, 8 threads")


def baseline_ratio(args, value):
    base = BASELINE_DECODE_TOKS.get((args.shape, args.ctx, args.batch))
    if base is None or args.layers != SHAPES[args.shape][1]:
        return None
    return round(value / base, 1)


def _cpu_flags():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("flags"):
                return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def reference_arm(args):
    """tkran2/bitwise itself, unmodified, on the same shape, batch and context.  It is a CMake
    C++ project for the CPU without a Python package to install, so its sources are copied
    beside the harness baseline/ref_bench.cpp into baseline/_ref/ and compiled there with its own
    flags (CMakeLists.txt:5-18: Release, -ffp-contract=off -fno-fast-math, AVX-512 where the CPU
    has it); the harness drives Model::random, Runner::forward and argmax_row."""
    import shutil
    unavailable = lambda why: {"impl": "reference", "unavailable": why}
    ref = os.path.join(HERE, "baseline", "_ref")
    src = os.path.join(ref, "src")
    names = ("kernels.cpp", "model.cpp", "engine.cpp", "block_manager.cpp")
    if not all(os.path.isfile(os.path.join(src, f)) for f in names):
        origin = os.path.join(REFERENCE_SOURCE, "src")
        if not os.path.isdir(origin):
            return unavailable("the reference's sources are neither in baseline/_ref/src nor at " + REFERENCE_SOURCE)
        os.makedirs(ref, exist_ok=True)
        shutil.copytree(origin, src, dirs_exist_ok=True)
    cxx = shutil.which("g++") or shutil.which("c++")
    flags = _cpu_flags()
    avx = {"avx512f", "avx512bw", "avx512vl", "fma"} <= flags
    exe = os.path.join(ref, "ref_bench_avx512" if avx else "ref_bench_scalar")
    harness = os.path.join(HERE, "baseline", "ref_bench.cpp")
    newest = max(os.path.getmtime(os.path.join(src, f)) for f in os.listdir(src))
    if not os.path.isfile(exe) or os.path.getmtime(exe) < max(newest, os.path.getmtime(harness)):
        if not cxx:
            return unavailable("no C++ compiler on this machine (g++, c++) to build the reference with")
        cmd = [cxx, "-std=c++20", "-O3", "-DNDEBUG", "-ffp-contract=off", "-fno-fast-math", "-pthread"]
        cmd += ["-mavx512f", "-mavx512bw", "-mavx512vl", "-mfma"] if avx else []
        cmd += ["-I", src, harness, *[os.path.join(src, f) for f in names], "-o", exe]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            return unavailable("the reference does not compile here: " + r.stderr.strip().split("\n")[-1][:200])
    title, full_layers, kw, shape_ctx = SHAPES[args.shape]
    layers = args.layers or full_layers
    ctx = args.ctx or shape_ctx
    warmup = max(3, args.warmup)
    threads = min(os.cpu_count() or 8, 64)
    points = [] if args.skip_points else [b for b in (1, 64) if b != args.batch]
    cmd = [exe, layers, kw["hidden_size"], kw["num_attention_heads"], kw["num_key_value_heads"], kw["head_dim"],
           kw["intermediate_size"], kw["vocab_size"], kw["rope_theta"], threads, ctx, args.batch, args.steps, warmup,
           0 if args.skip_prefill else 2048, *points]
    try:
        r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True, timeout=3000)
    except subprocess.TimeoutExpired:
        return unavailable("the reference did not finish the workload within 50 minutes on this machine's CPU")
    if r.returncode != 0:
        return unavailable(f"the reference's harness ended with code {r.returncode}: {r.stderr.strip()[-200:]}")
    out = json.loads(r.stdout.strip().split("\n")[-1])
    ms = out["ms_per_step"]
    value = args.batch / (ms / 1e3)
    line = {
        "metric": f"decode tok/s at batch {args.batch}, {ctx:,}-token context ({title})",
        "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 weights, fp32 compute (the reference's serving mode)",
        "data": "synthetic: the reference's Model::random weights, zero-filled cache, fixed token ids",
        "impl": "reference",
        "config": {"model": title, "layers": full_layers, "layers_run": layers, "hidden": kw["hidden_size"],
                   "heads": kw["num_attention_heads"], "kv_heads": kw["num_key_value_heads"], "head_dim": kw["head_dim"],
                   "intermediate": kw["intermediate_size"], "vocab": kw["vocab_size"], "global_batch": args.batch,
                   "seq_len": ctx, "page_size": 16, "parallelism": f"CPU, {threads} threads",
                   "build": "AVX-512" if avx else "portable scalar path (this CPU lacks AVX-512)",
                   "api": "bw::Model::random, bw::Runner::forward, bw::argmax_row", "timing": "host clock"},
        "clocks": {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["runs on the CPU"]},
        "gpu_launches": 0,
        "e2e": {"value": round(args.batch / (out["e2e_ms_per_step"] / 1e3), 2), "unit": "tokens/s",
                "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                "settings": "Runner::forward plus the reference's greedy sampler, host tokens in and out"},
    }
    if "prefill_ms" in out:
        line["prefill"] = {"value": round(2048 / (out["prefill_ms"] / 1e3), 2), "tokens": 2048, "ms": out["prefill_ms"]}
    pts = {f"decode_b{b}": round(b / (out[f"decode_b{b}_ms"] / 1e3), 2) for b in points if f"decode_b{b}_ms" in out}
    if pts:
        line["points"] = pts
    return line


def run_serve(model, title, args, pk):
    """Continuous batching through the engine: 64 requests, prompt lengths uniform in [16, 1024],
    output lengths uniform in [16, 256], prompts cut under a 512-token budget; host clock around
    the whole run, which is repeated after one untimed pass."""
    import numpy as np
    import torch
    from bitwise_b200 import Engine, EngineConfig, SamplingParams
    c = model.config
    rng = np.random.default_rng(3)
    n = 64
    plen = rng.integers(16, 1025, n)
    olen = rng.integers(16, 257, n)
    prompts = [rng.integers(0, c.vocab_size, int(l)).tolist() for l in plen]
    params = [SamplingParams(temperature=0.0, max_new_tokens=int(o), ignore_eos=True) for o in olen]
    page = args.page
    blocks = sum((int(p) + int(o) + page) // page for p, o in zip(plen, olen)) + 8
    out = {}
    with ClockSampler() as clocks:
        for rep in range(2):
            eng = Engine(model, EngineConfig(num_blocks=blocks, block_size=page, max_batched_tokens=512,
                                             max_num_seqs=n, fingerprint_logits=False, max_model_len=2048))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            res = eng.generate(prompts, params)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            made = sum(len(r) for r in res)
            out = {"value": made / dt, "seconds": dt, "steps": eng.stats.steps, "generated": made,
                   "prompt_tokens": int(plen.sum()), "launches": model.ops.launches,
                   "graph_replays": eng.stepper.graph_replays, "preemptions": eng.stats.preemptions}
            del eng
            torch.cuda.empty_cache()
    # what the crowd generated must be what each request generates alone (the reference's oracle,
    # sim/simulate.cpp:102-118): five of the requests are run again, each on an idle engine
    checked, wrong = 0, 0
    for i in (0, 13, 27, 41, 63):
        solo = Engine(model, EngineConfig(num_blocks=(int(plen[i]) + int(olen[i]) + page) // page + 1, block_size=page,
                                          max_batched_tokens=512, max_num_seqs=1, fingerprint_logits=False))
        checked += 1
        wrong += int(solo.generate([prompts[i]], [params[i]])[0] != res[i])
        del solo
    return {
        "metric": f"generated tok/s, 64 mixed requests under a 512-token budget ({title})",
        "value": round(out["value"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": out["steps"], "warmup": 1,
        "ms_per_step": round(out["seconds"] * 1e3 / max(1, out["steps"]), 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: random N(0,0.02) weights, prompt ids uniform over the vocabulary", "impl": "ours",
        "config": {"model": title, "layers": c.num_hidden_layers, "hidden": c.hidden_size,
                   "heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate": c.intermediate_size, "vocab": c.vocab_size, "requests": n,
                   "prompt_tokens": out["prompt_tokens"], "generated_tokens": out["generated"],
                   "token_budget": 512, "page_size": page, "parallelism": "single GPU",
                   "timing": "host clock around Engine.generate, second of two passes",
                   "steps_replayed_as_graphs": out["graph_replays"], "preemptions": out["preemptions"],
                   "requests_checked_against_solo_runs": checked, "requests_that_differ": wrong},
        "clocks": clocks.summary(), "gpu_launches": out["launches"],
        "total_tokens_per_s": round((out["prompt_tokens"] + out["generated"]) / out["seconds"], 1),
    }


if __name__ == "__main__":
    sys.exit(main())
