"""Decode-step benchmark of the hybrid cache path (SpikingBrain-7B shapes) on B200.

One step = one decode token for every sequence of the batch through the cache path of all
28 layers of the 7B model: 14 sliding-window layers (paged-KV append + block retirement,
then sliding-window paged attention, through MetaAttentionImpl.forward) and 14 GLA layers
(in-place recurrent-state step + read-out, through my_fused_recurrent_gla). The dense
projections / MLP of the model are the callers of this path and are not part of it.

Workload (per GPU): batch 256, every sequence at 8192 tokens of context, window 4096
(window_left 4096: the query plus 4096 keys, the vLLM-side convention of the reference),
28 query / 4 kv heads, head_dim 128, bf16 K/V in 16-token blocks behind a randomly
permuted block table, fp32 GLA state [256, 28, 128, 128] per layer. Synthetic data.
N GPUs: every rank owns its own 256 sequences (sequence sharding, no collective) -> weak scaling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--batch B] [--ctx L]

Prints ONE JSON line (rank 0). `--impl reference` times the CPU oracle (the PyTorch
restatement of the reference path) on the host cores instead.

The default run is the configuration the metric is quoted on (batch 256 at 8192 tokens). The other
configurations of the path have lines of their own (never the headline):
    --config 2     single-step op test: one sliding-window + one GLA layer, batch 64, contexts
                   uniform in [1024, 32768]
    --config 4     long-context eviction: per GPU one 131072-token prompt prefilled in 8192-token
                   chunks through the block tables (append + windowed attention + GLA scan), then
                   512 decode steps, on the device-resident planner
    --head-shard   churn shapes (1024 sequences, Zipf lengths) with the heads split over the ranks
`--full-step` adds to the default line the same step with the model's dense callers around the
path (projections, MLP, norms, logits: plain PyTorch on random bf16 weights of the 7B shapes), as
`full_step`, so that the cache-path tokens/s is not read as a model throughput.
"""
import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, KVH, D, WINDOW_LEFT, BLOCK = 28, 4, 128, 4096, 16
N_SWA, N_GLA = 14, 14
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes moved per algorithmic byte by the sliding-window decode kernel: a constant taken from
# one ncu capture of one launch at this batch and context (dram__bytes_read.sum 2.1582 GB +
# dram__bytes_write.sum 6.5 MB for 2.1481 GB of visible K/V: no re-reads), not measured in this
# run. Traffic grows in proportion to the tokens read.
SWA_TRAFFIC_PER_ALGORITHMIC_BYTE = (2.158249e9 + 6.497536e6) / (256 * 4097 * 2048)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=None,
                    help="sequences per GPU (default: 256; --config 2: 64; --config 4: 1)")
    ap.add_argument("--ctx", type=int, default=8192, help="context length of every sequence")
    ap.add_argument("--swa-layers", type=int, default=N_SWA)
    ap.add_argument("--gla-layers", type=int, default=N_GLA)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--head-shard", action="store_true",
                    help="instead of the headline run: the churn workload (1024 sequences, Zipf lengths) with attention "
                         "heads split over the ranks, sliding-window decode + gather of the head outputs per layer")
    ap.add_argument("--config", type=int, default=3, choices=[2, 3, 4],
                    help="which configuration of the path to run (3 = the headline; 2 and 4 print lines of their own)")
    ap.add_argument("--full-step", action="store_true",
                    help="also time the decode step with the model's dense callers (plain PyTorch) around the path")
    ap.add_argument("--prompt", type=int, default=131072, help="--config 4: prompt tokens per sequence")
    ap.add_argument("--chunk", type=int, default=8192, help="--config 4: prefill chunk")
    ap.add_argument("--decode-steps", type=int, default=512, help="--config 4: decode steps after the prompt")
    ap.add_argument("--tp", type=int, default=0,
                    help="--head-shard: head shards per group (default: all ranks); the ranks form world/tp "
                         "sequence groups, e.g. 8 GPUs as 4 head shards x 2 groups")
    args = ap.parse_args()
    if args.batch is None:
        args.batch = {2: 64, 3: 256, 4: 1}[args.config]
    if args.config == 2:
        args.swa_layers = args.gla_layers = 1
    return args


# ------------------------------------------------------------------------- bytes model
def cache_bytes_per_step(lens_after, n_swa, n_gla):
    """Algorithmic cache bytes of one decode step (K/V read + appended, GLA state read+written) for
    sequences of the given lengths (after the step's token)."""
    batch = len(lens_after)
    vis = sum(min(int(L), WINDOW_LEFT + 1) for L in lens_after)
    swa = vis * 2 * KVH * D * 2 + batch * 2 * KVH * D * 2
    gla = batch * 2 * H * D * D * 4
    return n_swa * swa + n_gla * gla, swa, gla


def config_lens(args):
    """Context length of every sequence of a rank at the start of the run."""
    import numpy as np
    if args.config == 2:      # uniform in [1024, 32768], seed 0
        return np.random.default_rng(0).integers(1024, 32769, size=args.batch).astype(np.int64)
    return np.full(args.batch, args.ctx, dtype=np.int64)


# ------------------------------------------------------------------- CPU oracle timing
def cpu_reference_step_seconds(n_seqs, ctx, repeats):
    """Seconds the CPU restatement of the reference path needs for ONE sliding-window layer
    plus ONE GLA layer on `n_seqs` sequences at context `ctx` (median of `repeats`):
    Cache.update window roll + repeat_kv + masked softmax attention (the HF path), and the
    fp32 recurrence on a fresh state tensor."""
    import torch
    from oracle import ref_ops
    torch.manual_seed(0)
    W = WINDOW_LEFT  # the HF cache keeps `window` tokens
    n_cached = min(ctx, W)
    cache = ref_ops.RefWindowCache()
    k0 = (torch.randn(n_seqs, KVH, n_cached, D) / math.sqrt(D)).bfloat16()
    v0 = (torch.randn(n_seqs, KVH, n_cached, D) / math.sqrt(D)).bfloat16()
    cache.update(attn_state=(k0, v0), layer_idx=0, offset=n_cached, cache_kwargs={"window_size": W})
    q = (torch.randn(n_seqs, H, D) / math.sqrt(D)).bfloat16()
    kn = (torch.randn(n_seqs, KVH, 1, D) / math.sqrt(D)).bfloat16()
    gq, gk, gg = ref_ops.gla_prepare_inputs(torch.randn(n_seqs, H, D), torch.randn(n_seqs, KVH, D),
                                            torch.randn(n_seqs, KVH, D))
    gv = torch.randn(n_seqs, KVH, D)
    state = torch.randn(n_seqs, H, D, D)
    times = []
    for it in range(repeats + 1):
        t0 = time.perf_counter()
        st = cache.update(attn_state=(kn, kn), layer_idx=0, offset=1, cache_kwargs={"window_size": W})
        kc, vc = st["attn_state"]
        for b in range(n_seqs):
            ref_ops.swa_decode_ref(q[b], kc[b], vc[b], D ** -0.5, window=W)
        ref_ops.gla_step_ref(gq, gk, gv, gg, state)
        dt = time.perf_counter() - t0
        if it > 0:
            times.append(dt)
    return statistics.median(times)


def use_all_host_threads():
    """Launchers such as torch.distributed.run pin OMP_NUM_THREADS to 1; the CPU arm is meant to
    use every core the box has."""
    import torch
    n = os.cpu_count() or 1
    if torch.get_num_threads() < n:
        torch.set_num_threads(n)
    return torch.get_num_threads()


def cpu_baseline(args, sample_seqs=8, repeats=5):
    cores = use_all_host_threads()
    t = cpu_reference_step_seconds(sample_seqs, args.ctx + 1, repeats)
    per_seq_layerpair = t / sample_seqs
    # a full step = batch sequences x (swa_layers + gla_layers); the sample timed one of each
    pairs = max(args.swa_layers, args.gla_layers)
    step_s = per_seq_layerpair * args.batch * pairs
    return {
        "value": args.batch / step_s, "unit": "tokens/s", "cores": cores, "kind": "port",
        "sample": f"{sample_seqs} sequences x (1 sliding-window layer + 1 GLA layer) at ctx {args.ctx + 1}, "
                  f"median of {repeats}, scaled x{args.batch / sample_seqs:g} sequences x{pairs} layer pairs",
    }


# --------------------------------------------------------------------- clocks sampling
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.Q}",
                 "--format=csv,noheader,nounits", "-lms", "50"], stdout=f, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        with open(self.path) as f:
            for line in f:
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1])); smax.append(float(p[2]))
                except ValueError:
                    continue
                for nm, val in zip(names, p[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------ instrumentation
class Instrument:
    """The benchmark's own bookkeeping around the library calls it goes through (the library
    carries none): `launches` counts the kernels launched through spikingbrain_7b_b200.ops, and
    while `timing` is a list every swa_decode call appends a (start, end) pair of CUDA events
    recorded on the launching stream around its kernel. Installed by wrapping the functions of
    the ops module once per process."""
    _installed = None

    def __init__(self, ops, abi):
        import torch
        self.launches = 0
        self.timing = None
        count = {
            "kv_append": lambda a, kw: 1, "rope_kv_append": lambda a, kw: 1, "kv_gather": lambda a, kw: 1,
            "swa_decode": lambda a, kw: -(-a[0].shape[0] // 1024), "gla_step": lambda a, kw: 1,
            "swa_prefill": lambda a, kw: 1, "swa_prefill_dense": lambda a, kw: 1, "plan_step": lambda a, kw: 1,
            "release_rows": lambda a, kw: 1,
            "gla_scan": self._scan_launches,
        }
        for name, n_of in count.items():
            inner = getattr(ops, name)

            def wrapped(*a, _inner=inner, _n=n_of, _name=name, **kw):
                timing = self.timing if _name == "swa_decode" else None
                if timing is not None:
                    # external: inside a stream capture these become event-record nodes of the
                    # graph, so the pair times the launch of the latest replay
                    ev0 = torch.cuda.Event(enable_timing=True, external=True)
                    ev1 = torch.cuda.Event(enable_timing=True, external=True)
                    ev0.record()
                out = _inner(*a, **kw)
                if timing is not None:
                    ev1.record()
                    timing.append((ev0, ev1))
                self.launches += _n(a, kw)
                return out

            setattr(ops, name, wrapped)

    def _scan_launches(self, a, kw):
        """Kernels one gla_scan call launches: one chain per (sequence, head); the tensor-core form plus the
        token-by-token kernel that finishes what it left; or local scans + carry + scan proper."""
        import torch
        from spikingbrain_7b_b200 import _abi
        mql = int(kw.get("max_query_len", 0))
        if kw.get("workspace") is None or mql <= 0:
            return 1
        n_seqs, H, D = a[5].numel() - 1, a[0].shape[1], a[0].shape[2]
        hand_over = (2 * n_seqs * H * 4 + 255) // 256 * 256 if mql >= 256 else 0
        if hand_over and a[0].dtype == torch.bfloat16 and D == 128:
            # tensor-core form + the token-by-token kernel behind it; with few chains: local pass, carry
            # (three pieces or more) and full pass
            chains, n_chunks = n_seqs * H, -(-mql // 128)
            if 2 * chains <= 148 and n_chunks >= 4:
                per = max(2, -(-n_chunks // (148 // chains)))
                n_sub = -(-n_chunks // per)
                if n_sub >= 2:
                    return 3 + (1 if n_sub > 2 else 0)
            return 2
        return 3 if _abi.lib.sbk_gla_scan_workspace_bytes(n_seqs, mql, H, D) > hand_over else 1

    @classmethod
    def install(cls):
        if cls._installed is None:
            from spikingbrain_7b_b200 import _abi, ops
            cls._installed = cls(ops, _abi)
        return cls._installed


# -------------------------------------------------------------------------- the engine
class DecodeEngine:
    """Holds the per-layer caches of one GPU and runs decode steps through the reference-facing
    surfaces: MetaAttentionImpl.forward for sliding-window layers, my_fused_recurrent_gla for
    GLA layers. Lengths, block tables, the free-block ring and the step's slot mapping live on the
    GPU (DeviceStepPlanner): one sbk_plan_step launch per step stands in for the serving engine's
    block manager and metadata builder, so a step needs no host-side metadata work."""

    def __init__(self, args, device):
        import numpy as np
        import torch
        from spikingbrain_7b_b200 import ops
        from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
        from spikingbrain_7b_b200.block_pool import DeviceStepPlanner
        from spikingbrain_7b_b200.gla_slots import GLACacheManager, my_fused_recurrent_gla
        self.torch, self.np, self.ops = torch, np, ops
        self.instr = Instrument.install()
        self.Meta = MetaAttentionMetadata
        self.gla_fn = my_fused_recurrent_gla
        self.device = device
        self.B = B = args.batch
        self.n_swa, self.n_gla = args.swa_layers, args.gla_layers
        lens = config_lens(args)
        self.lens0 = lens
        total_steps = args.steps * 3 + args.warmup * 3 + 16
        max_len = int(lens.max()) + total_steps + 1
        self.max_blocks = (max_len + BLOCK - 1) // BLOCK + 1
        # sequences arrive with their context: only the window's blocks are resident, handed out
        # in a random order; the rest of the pool (three spare blocks per sequence) is the free ring
        first_live = np.maximum(0, lens - WINDOW_LEFT) // BLOCK
        last = (lens + BLOCK - 1) // BLOCK
        n_live = last - first_live
        n_blocks = int(n_live.sum()) + 3 * B + 64
        self.plan = DeviceStepPlanner(n_blocks, BLOCK, WINDOW_LEFT, B, self.max_blocks, device)
        g = np.random.default_rng(1234 + (device.index or 0))
        order = g.permutation(n_blocks).astype(np.int32)
        table = np.full((B, self.max_blocks), -1, dtype=np.int32)
        used = 0
        for b in range(B):
            table[b, first_live[b]:last[b]] = order[used:used + n_live[b]]
            used += int(n_live[b])
        self.plan.load_state(lens.astype(np.int32), table, order[used:])
        self.ctx0, self.steps_done = int(lens.max()), 0
        self.table_d, self.lens_d, self.slots_d = self.plan.block_tables, self.plan.seq_lens, self.plan.slot_mapping
        self.kv = []
        for _ in range(self.n_swa):
            t = torch.empty(2, n_blocks, BLOCK, KVH, D, dtype=torch.bfloat16, device=device)
            t.normal_(0.0, 1.0 / math.sqrt(D))
            self.kv.append(t)
        self.gla = GLACacheManager(torch.float32, (max(self.n_gla, 1), B, H, D, D), device=device)
        self.gla.cache.normal_(0.0, 1.0)
        _, self.slot_idx = self.gla.current_run_tensors({f"r{i}": [0] for i in range(B)})
        self.impls = [MetaAttentionImpl(H, D, D ** -0.5, KVH, None, WINDOW_LEFT + 1, "auto")
                      for _ in range(self.n_swa)]
        # layer inputs (what the projections of the model would hand over), device resident
        rn = lambda *s: (torch.randn(*s, device=device) / math.sqrt(D)).bfloat16()
        self.q = [rn(B, H, D) for _ in range(2)]
        self.k = [rn(B, KVH, D) for _ in range(2)]
        self.v = [rn(B, KVH, D) for _ in range(2)]
        self.gq = torch.relu(rn(B, H, 1, D))
        self.gk = torch.relu(rn(B, KVH, 1, D))
        self.gv = rn(B, KVH, 1, D)
        self.gg = (torch.nn.functional.logsigmoid(torch.randn(B, KVH, 1, D, device=device)) / 16).bfloat16()
        self.out = torch.empty(B, H, D, dtype=torch.bfloat16, device=device)
        self.gla_out = torch.empty(B, H, D, dtype=torch.bfloat16, device=device)
        self.graph = self.graph_e2e = self._e2e = self.graph_full = self._full = None
        self.swa_events = []
        self.launches_per_step = 0
        # pinned host staging for the end-to-end mode
        pin = lambda t: t.cpu().pin_memory()
        self.h_q, self.h_k, self.h_v = pin(self.q[0]), pin(self.k[0]), pin(self.v[0])
        self.h_gq, self.h_gk, self.h_gv, self.h_gg = pin(self.gq), pin(self.gk), pin(self.gv), pin(self.gg)
        self.h2d_bytes = self.d2h_bytes = 0
        self.e2e_in_bytes = self.e2e_out_bytes = 0

    def _metadata(self):
        """The step's metadata object: views of the planner's device tensors (fixed addresses)."""
        return self.Meta(num_prefills=0, num_prefill_tokens=0, num_decode_tokens=self.B,
                         slot_mapping=self.slots_d, seq_lens=None, seq_lens_tensor=self.lens_d,
                         max_prefill_seq_len=0, max_decode_seq_len=self.ctx0 + self.steps_done + 1,
                         context_lens_tensor=None, block_tables=self.table_d, use_cuda_graph=False,
                         max_query_len=1, max_decode_query_len=1)

    # ---------------------------------------------------------------- device-resident step
    def enqueue_layers(self, meta, timing=None):
        """All kernels of one decode step on the current stream, through the reference-facing
        calls. `timing`: list that receives an (start, end) event pair around every sliding-window
        decode call (events created with external=True so that a captured graph records them)."""
        torch, ops = self.torch, self.ops
        self.plan.plan()   # retire, allocate, slots, lengths: on the device
        for i in range(max(self.n_swa, self.n_gla)):
            if i < self.n_gla:   # even layers of the model are GLA layers
                self.gla_fn(self.gq, self.gk, self.gv, self.gg, kv_caches=self.gla.cache[i], slot_idx=self.slot_idx,
                            out=self.gla_out)
            if i < self.n_swa:   # odd layers are sliding-window layers
                j = i & 1
                # three of the sliding-window launches carry timing events (first, middle, last layer):
                # an event node between two kernels costs the overlap of their tail and head
                self.instr.timing = timing if i in (0, self.n_swa // 2, self.n_swa - 1) else None
                self.impls[i].forward(None, self.q[j], self.k[j], self.v[j], None, None, None, self.kv[i],
                                      meta, output=self.out)
                self.instr.timing = None

    def step(self, e2e=False):
        """One decode step: the planner launch and the layers' kernels -- replayed from a captured
        CUDA graph once `capture()` was called, launched one by one before that."""
        meta = self._metadata()
        self.steps_done += 1
        if e2e:
            if self.graph_e2e is not None:
                self.graph_e2e.replay()
                self.h2d_bytes += self.e2e_in_bytes
                self.d2h_bytes += self.e2e_out_bytes
                self.torch.cuda.current_stream().synchronize()
            else:
                self._enqueue_e2e(meta)
                self._e2e.done.synchronize()
            # either way the caller now holds every layer output of the step on the host
        elif self.graph is not None:
            self.graph.replay()
        else:
            self.enqueue_layers(meta)

    def capture(self, e2e=False):
        """Capture the kernels (and, end to end, the host<->device copies) of one step into a CUDA
        graph. The metadata tensors the graph reads (slots, lengths, block table) live at fixed
        addresses and are advanced by the graph's own first node."""
        torch, ops = self.torch, self.ops
        meta = self._metadata()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            if e2e:
                self._e2e_setup()
                self._enqueue_e2e(meta)             # warm-up of the multi-stream pattern on the side stream
                side.wait_event(self._e2e.done)
                self.h2d_bytes = self.d2h_bytes = 0
                with torch.cuda.graph(g, stream=side):
                    self._enqueue_e2e(meta)
                self.e2e_in_bytes, self.e2e_out_bytes = self.h2d_bytes, self.d2h_bytes
                self.graph_e2e = g
            else:
                self.enqueue_layers(meta)
                launches0 = self.instr.launches
                self.swa_events = []
                with torch.cuda.graph(g, stream=side):
                    self.enqueue_layers(meta, timing=self.swa_events)
                self.launches_per_step = self.instr.launches - launches0
                self.graph = g
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()

    # ---------------------------------------------------- the step with the model's dense callers
    HIDDEN, INTER, VOCAB = 3584, 18944, 152064

    def _full_setup(self):
        """Random bf16 weights of the 7B shapes (hidden 3584, MLP 18944, 28 layers alternating GLA /
        sliding-window attention, vocabulary 152064): the callers of the cache path, as plain PyTorch."""
        torch = self.torch
        if self._full is not None:
            return self._full
        dev, hid, inter = self.device, self.HIDDEN, self.INTER
        kvd = KVH * D

        def w(o, i):
            return torch.empty(o, i, device=dev, dtype=torch.bfloat16).normal_(0.0, i ** -0.5)

        ones = lambda n: torch.ones(n, device=dev, dtype=torch.bfloat16)
        f = type("Full", (), {})()
        f.gla, f.swa = [], []
        mlp = lambda: dict(n2=ones(hid), gate_up=w(2 * inter, hid), down=w(hid, inter))
        for _ in range(self.n_gla):
            f.gla.append(dict(n1=ones(hid), qkv=w(hid + 2 * kvd, hid), gk0=w(16, hid), gk1=w(kvd, 16), gate=w(hid, hid),
                              o=w(hid, hid), g_norm=ones(D), **mlp()))
        for _ in range(self.n_swa):
            f.swa.append(dict(n1=ones(hid), qkv=w(hid + 2 * kvd, hid), o=w(hid, hid), **mlp()))
        f.final_norm, f.lm_head = ones(hid), w(self.VOCAB, hid)
        f.x0 = torch.randn(self.B, hid, device=dev).bfloat16()
        f.tokens = torch.zeros(self.B, dtype=torch.int64, device=dev)
        f.attn_out = torch.empty(self.B, H, D, dtype=torch.bfloat16, device=dev)
        f.cos_sin = self.ops.build_cos_sin_cache(D, self.max_blocks * BLOCK, 1e6, torch.bfloat16, dev)
        n_params = sum(t.numel() for lay in f.gla + f.swa for t in lay.values()) + f.lm_head.numel()
        f.weight_bytes = 2 * n_params
        self._full = f
        return f

    def enqueue_full(self, meta):
        """One decode step of the whole stack on the current stream: norms, projections, the cache path
        (GLA step with its fused neighbours; rotary + append + sliding-window decode), output
        projections, MLPs and the logits' argmax. The dense parts are torch ops (cuBLAS)."""
        from spikingbrain_7b_b200.gla_slots import gla_decode_layer
        torch, f = self.torch, self._full_setup()
        F = torch.nn.functional
        hid, inter, kvd, B = self.HIDDEN, self.INTER, KVH * D, self.B
        self.plan.plan()
        h = f.x0

        def mlp(h, lay):
            r = F.rms_norm(h, (hid,), lay["n2"], 1e-6)
            gu = r @ lay["gate_up"].t()
            return h + (F.silu(gu[:, :inter]) * gu[:, inter:]) @ lay["down"].t()

        for i in range(max(self.n_swa, self.n_gla)):
            if i < self.n_gla:
                lay = f.gla[i]
                r = F.rms_norm(h, (hid,), lay["n1"], 1e-6)
                qkv = r @ lay["qkv"].t()
                q = qkv[:, :hid].reshape(B, H, D)
                k = qkv[:, hid:hid + kvd].reshape(B, KVH, D)
                v = qkv[:, hid + kvd:].reshape(B, KVH, D)
                gk = ((r @ lay["gk0"].t()) @ lay["gk1"].t()).view(B, KVH, D)
                o = gla_decode_layer(q, k, v, gk, self.gla.cache[i], self.slot_idx, lay["g_norm"])
                o = o.view(B, hid) * F.silu(r @ lay["gate"].t())
                h = mlp(h + o @ lay["o"].t(), lay)
            if i < self.n_swa:
                lay = f.swa[i]
                r = F.rms_norm(h, (hid,), lay["n1"], 1e-6)
                qkv = r @ lay["qkv"].t()
                q = qkv[:, :hid].view(B, H, D)
                k = qkv[:, hid:hid + kvd].view(B, KVH, D)
                v = qkv[:, hid + kvd:].view(B, KVH, D)
                self.impls[i].forward(None, q, k, v, None, None, None, self.kv[i], meta, output=f.attn_out,
                                      positions=self.plan.positions, cos_sin_cache=f.cos_sin)
                h = mlp(h + f.attn_out.view(B, hid) @ lay["o"].t(), lay)
        logits = F.rms_norm(h, (hid,), f.final_norm, 1e-6) @ f.lm_head.t()
        f.tokens.copy_(logits.argmax(-1))

    def capture_full(self):
        torch = self.torch
        meta = self._metadata()
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            self.enqueue_full(meta)          # warm-up: cuBLAS workspaces, kernel attributes
            self.enqueue_full(meta)
            with torch.cuda.graph(g, stream=side):
                self.enqueue_full(meta)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.steps_done += 3
        self.graph_full = g

    def step_full(self):
        self.steps_done += 1
        self.graph_full.replay()

    # ------------------------------------------------------------------- end-to-end step
    def _e2e_setup(self):
        """Double-buffered device inputs/outputs, one stream per copy direction, and the events
        that order them against the compute stream."""
        torch = self.torch
        if self._e2e is not None:
            return self._e2e
        dev = self.device
        ev = lambda: torch.cuda.Event()
        st = type("E2E", (), {})()
        st.h2d, st.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        st.g_in = [[torch.empty_like(t) for t in (self.gq, self.gk, self.gv, self.gg)] for _ in range(2)]
        st.s_in = [[self.q[j], self.k[j], self.v[j]] for j in range(2)]
        st.out = [torch.empty_like(self.out) for _ in range(2)]
        st.h_out = [torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory() for _ in range(2)]
        st.in_ready = {k: [ev(), ev()] for k in "gs"}     # recorded on h2d: inputs of slot landed
        st.in_free = {k: [ev(), ev()] for k in "gs"}      # recorded on compute: slot consumed
        st.out_ready, st.out_free = [ev(), ev()], [ev(), ev()]
        st.done = ev()
        self._e2e = st
        return st

    def _enqueue_e2e(self, meta):
        """One step as a caller with HOST buffers sees it: every layer's inputs travel from pinned
        host memory (H2D stream, a layer ahead of the math), every layer's output travels back
        (D2H stream); `done` fires when the last output is on the host."""
        torch, ops = self.torch, self.ops
        st = self._e2e_setup()
        cur = torch.cuda.current_stream()
        self.plan.plan()
        for k in "gs":                      # every buffer starts the step free
            for e in st.in_free[k]:
                e.record(cur)
        for e in st.out_free:
            e.record(cur)
        n_out = 0

        def upload(kind, slot, pairs):
            st.h2d.wait_event(st.in_free[kind][slot])
            with torch.cuda.stream(st.h2d):
                for dst, src in pairs:
                    dst.copy_(src, non_blocking=True)
                    self.h2d_bytes += src.numel() * src.element_size()
            st.in_ready[kind][slot].record(st.h2d)
            cur.wait_event(st.in_ready[kind][slot])

        def download(o, oslot):
            st.out_ready[oslot].record(cur)
            st.d2h.wait_event(st.out_ready[oslot])
            with torch.cuda.stream(st.d2h):
                st.h_out[oslot].copy_(o, non_blocking=True)
            st.out_free[oslot].record(st.d2h)
            self.d2h_bytes += o.numel() * o.element_size()

        for i in range(max(self.n_swa, self.n_gla)):
            slot = i & 1
            if i < self.n_gla:
                gi = st.g_in[slot]
                upload("g", slot, zip(gi, (self.h_gq, self.h_gk, self.h_gv, self.h_gg)))
                oslot = n_out & 1; n_out += 1
                cur.wait_event(st.out_free[oslot])      # its previous content is on the host
                self.gla_fn(gi[0], gi[1], gi[2], gi[3], kv_caches=self.gla.cache[i], slot_idx=self.slot_idx,
                            out=st.out[oslot])
                st.in_free["g"][slot].record(cur)
                download(st.out[oslot], oslot)
            if i < self.n_swa:
                q, k, v = st.s_in[slot]
                upload("s", slot, zip((q, k, v), (self.h_q, self.h_k, self.h_v)))
                oslot = n_out & 1; n_out += 1
                cur.wait_event(st.out_free[oslot])
                self.impls[i].forward(None, q, k, v, None, None, None, self.kv[i], meta, output=st.out[oslot])
                st.in_free["s"][slot].record(cur)
                download(st.out[oslot], oslot)
        cur.wait_stream(st.h2d)             # join both copy streams (needed when this is captured)
        cur.wait_stream(st.d2h)
        st.done.record(cur)


# ------------------------------------------------------------------- multi-rank plumbing
def dist_setup(backend, device=None):
    """(rank, world); joins the process group when launched with more than one rank."""
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world > 1 and not dist.is_initialized():
        if backend == "nccl":
            dist.init_process_group("nccl", device_id=device)
        else:
            dist.init_process_group(backend)
    return rank, world


def max_over_ranks(value, device):
    """The slowest rank's time: every rank works on its own sequences, the job ends with the last."""
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def workload_name(args):
    shapes = f"window_left {WINDOW_LEFT}, block {BLOCK}, 28/4 heads, head_dim 128"
    if args.config == 2:
        return (f"single-step op test: {args.swa_layers} sliding-window + {args.gla_layers} GLA layer, batch {args.batch} "
                f"per GPU, ctx uniform in [1024, 32768] (numpy default_rng(0)), {shapes}")
    return (f"7B-shaped decode step, cache path of {args.swa_layers} sliding-window + {args.gla_layers} GLA layers, "
            f"batch {args.batch} per GPU, ctx {args.ctx}, {shapes}")


def job_tokens_per_s(batch_per_rank, world, ms_per_step):
    """Whole-job throughput: every rank decodes one token for each of its sequences per step."""
    return batch_per_rank * world / (ms_per_step * 1e-3)


def run_b200(args):
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", 0))
    if int(os.environ.get("WORLD_SIZE", 1)) == 1 and args.gpus > 1:
        raise SystemExit("launch multi-GPU runs with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    rank, world = dist_setup("nccl", device)

    # builds the library on first use if needed (it normally travels prebuilt)
    import importlib.util
    spec = importlib.util.spec_from_file_location("_sb7b_build", os.path.join(ROOT, "spikingbrain-7b_b200", "build.py"))
    bmod = importlib.util.module_from_spec(spec); spec.loader.exec_module(bmod)
    if rank == 0:
        bmod.build_library()
    if world > 1:
        dist.barrier()

    from spikingbrain_7b_b200 import ops
    eng = DecodeEngine(args, device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    swa_ms = []

    def harvest():
        """Durations of the sliding-window decode launches of the step that just ran."""
        torch.cuda.synchronize()
        swa_ms.extend(a.elapsed_time(b) for a, b in eng.swa_events)

    def timed(n_steps, e2e, sample_every=0):
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for i in range(n_steps):
            eng.step(e2e=e2e)
            if sample_every and (i + 1) % sample_every == 0:
                harvest()
        e1.record()
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3
        ms = max(e0.elapsed_time(e1), 0.0)
        if e2e:
            ms = max(ms, wall)   # the host waits inside an end-to-end step; take the slower clock
        ms = max_over_ranks(ms, device)
        barrier()
        return ms

    # ---- device-resident timing ----
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()   # sampling starts with the warm-up: the tool needs a moment to come up
    for _ in range(max(args.warmup, 3)):
        eng.step()
    if args.no_graph:
        launches0 = eng.instr.launches
        timing = []
        _orig = eng.enqueue_layers
        eng.enqueue_layers = lambda meta, timing=timing: _orig(meta, timing=timing)
        total_ms = timed(args.steps, e2e=False)
        torch.cuda.synchronize()
        swa_ms.extend(a.elapsed_time(b) for a, b in timing)
        launches = eng.instr.launches - launches0
        eng.enqueue_layers = _orig
    else:
        eng.capture()
        eng.step()
        # every 10th step the launch timings of that replay are read back (one host sync each)
        total_ms = timed(args.steps, e2e=False, sample_every=10)
        launches = eng.launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = total_ms / args.steps

    # ---- end to end: host buffers in, host result out, every step ----
    e2e_obj = None
    if not args.no_e2e:
        for _ in range(3):
            eng.step(e2e=True)
        if not args.no_graph:
            eng.capture(e2e=True)
            eng.step(e2e=True)
        eng.h2d_bytes = eng.d2h_bytes = 0
        e2e_ms = timed(args.steps, e2e=True) / args.steps
        e2e_obj = {"value": job_tokens_per_s(args.batch, world, e2e_ms), "unit": "tokens/s",
                   "h2d_bytes_per_step": eng.h2d_bytes // args.steps,
                   "d2h_bytes_per_step": eng.d2h_bytes // args.steps, "ms_per_step": e2e_ms}

    # ---- the decode kernel alone: back-to-back launches over two copies of one layer's pool in turn
    #      (together larger than L2), no event nodes between graph kernels, nothing else running ----
    alone_ms = None
    if eng.n_swa:
        pools = [eng.kv[0], eng.kv[0].clone()]
        call = lambda i: eng.impls[0]._decode(eng.q[0], pools[i & 1], eng.table_d, eng.lens_d, WINDOW_LEFT, eng.out)
        for i in range(4):
            call(i)
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(20):
            call(i)
        e1.record()
        torch.cuda.synchronize()
        alone_ms = max_over_ranks(e0.elapsed_time(e1) / 20, device)
        del pools

    # ---- the same step with the model's dense callers around the path (plain PyTorch) ----
    full_obj = None
    if args.full_step:
        eng.capture_full()
        for _ in range(3):
            eng.step_full()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            eng.step_full()
        e1.record()
        torch.cuda.synchronize()
        full_ms = max_over_ranks(e0.elapsed_time(e1), device) / args.steps
        full_obj = {"tokens_per_s": job_tokens_per_s(args.batch, world, full_ms), "ms_per_step": full_ms,
                    "cache_path_share_of_step": ms_per_step / full_ms, "weight_bytes_per_gpu": eng._full.weight_bytes,
                    "what": "the decode step with RMSNorm, QKV / gate / low-rank gate / output projections, SwiGLU MLP "
                            "and logits + argmax as torch ops on random bf16 weights of the 7B shapes (hidden 3584, "
                            "MLP 18944, vocabulary 152064), the cache path through the fused forms (rotary in the append; "
                            "ReLU, gate and g_norm in the GLA step); CUDA graph replay"}

    # every status word of the run: the layers' kernels and the planner (a step the planner refuses
    # -- out of blocks, table full -- fills the slot mapping with -1 and appends nothing, so a run
    # that saw one has not timed the workload)
    status = 0
    for impl in eng.impls:
        status |= impl.status()
    status |= int(eng.plan.status.item())
    if status != 0:
        raise SystemExit(f"rank {rank}: device status {status} after the timed steps; the run is void")
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    lens_mid = eng.lens0 + max(args.warmup, 3) + args.steps // 2
    step_bytes, swa_layer_bytes, gla_layer_bytes = cache_bytes_per_step(lens_mid, args.swa_layers, args.gla_layers)
    swa_avg_ms = statistics.mean(swa_ms) if swa_ms else None
    achieved = swa_layer_bytes / (swa_avg_ms * 1e-3) / 1e9 if swa_avg_ms else None
    line = {
        "metric": "decode tokens/s and cache HBM GB/s (% of 8 TB/s)",
        "value": job_tokens_per_s(args.batch, world, ms_per_step), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 K/V, f32 GLA state",
        "data": "synthetic",
        "config": {"workload": workload_name(args),
                   "parallelism": f"sequence-sharded x{world}, no collective",
                   "launch": "host launches" if args.no_graph else "CUDA graph replay of the step (planner launch + layer kernels); no host metadata work",
                   "l2": f"the step streams {step_bytes / 1e6:.0f} MB of K/V and GLA state, more than the 126 MB L2; no flush needed"},
        "cache_gbs": world * step_bytes / (ms_per_step * 1e-3) / 1e9,
        "cache_gbs_per_gpu": step_bytes / (ms_per_step * 1e-3) / 1e9,
        "cache_frac_of_8tbs": step_bytes / (ms_per_step * 1e-3) / 1e9 / NOMINAL_HBM_GBS,
        "cache_bytes_per_step_per_gpu": step_bytes,
        "roofline": {"bound": "hbm", "kernel": "swa_decode_kernel (+ its split reduce)",
                     "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak if achieved else None, "peak_source": peak_src,
                     "frac_of_8tbs": achieved / NOMINAL_HBM_GBS if achieved else None,
                     "algorithmic_bytes_per_launch": swa_layer_bytes, "avg_launch_ms": swa_avg_ms,
                     "launches_timed": len(swa_ms),
                     "alone": {"avg_launch_ms": alone_ms,
                               "achieved": swa_layer_bytes / (alone_ms * 1e-3) / 1e9 if alone_ms else None,
                               "frac": swa_layer_bytes / (alone_ms * 1e-3) / 1e9 / peak if alone_ms else None,
                               "how": "20 back-to-back launches over two copies of one layer's pool in turn, nothing "
                                      "else on the GPU (inside the step a launch shares HBM with the write-back of the "
                                      "GLA kernel before it, and its timing events are graph nodes of their own)"},
                     "traffic": int(swa_layer_bytes * SWA_TRAFFIC_PER_ALGORITHMIC_BYTE),
                     "traffic_source": "constant from an ncu capture (dram__bytes_read.sum + dram__bytes_write.sum of "
                                       "one launch at this batch and context), scaled by tokens; not measured in this run"},
        "e2e": e2e_obj, "gpu_launches": launches, "clocks": clocks, "device_status": status,
    }
    if args.config == 2:
        line["gla_step_bytes_per_launch"] = gla_layer_bytes
    if full_obj is not None:
        line["full_step"] = full_obj
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(args)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_longctx(args):
    """Long-context eviction: every rank owns `batch` sequences (default one). A prompt of `--prompt`
    tokens goes through the path in chunks of `--chunk`: one planner launch per chunk (retire the blocks
    no token of the chunk can see, allocate the chunk's blocks, slots, lengths -- on the device), then per
    layer the GLA scan with state carry (chunk-parallel when the sequences are few) and, through
    MetaAttentionImpl.forward with prefill metadata, the append and the windowed attention over the block
    tables. Then `--decode-steps` one-token steps replayed from a CUDA graph. Sequence-sharded: no
    collective. Prints its own JSON line."""
    import numpy as np
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    rank, world = dist_setup("nccl", device)
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.backend import MetaAttentionImpl, MetaAttentionMetadata
    from spikingbrain_7b_b200.block_pool import DeviceStepPlanner
    from spikingbrain_7b_b200.gla_slots import GLACacheManager, gla_prefill_scan, my_fused_recurrent_gla
    instr = Instrument.install()
    S, prompt, chunk, dsteps = args.batch, args.prompt, args.chunk, args.decode_steps
    n_swa, n_gla = args.swa_layers, args.gla_layers
    if prompt % chunk:
        raise SystemExit("--prompt must be a multiple of --chunk")
    T = S * chunk
    max_blocks = (max(prompt, 2 * chunk) + dsteps) // BLOCK + 2      # (the warm-up below runs two chunks whatever the prompt)
    per_seq = (WINDOW_LEFT + chunk) // BLOCK + 4       # the window, the chunk in flight, partial blocks at the ends
    n_blocks = S * per_seq + 16
    plan = DeviceStepPlanner(n_blocks, BLOCK, WINDOW_LEFT, S, max_blocks, device, max_tokens=T)
    kv = [torch.zeros(2, n_blocks, BLOCK, KVH, D, dtype=torch.bfloat16, device=device) for _ in range(n_swa)]
    gla = GLACacheManager(torch.float32, (max(n_gla, 1), S, H, D, D), device=device)
    _, slot_idx = gla.current_run_tensors({f"r{i}": [0] for i in range(S)})
    impls = [MetaAttentionImpl(H, D, D ** -0.5, KVH, None, WINDOW_LEFT + 1, "auto") for _ in range(n_swa)]
    rn = lambda *s: (torch.randn(*s, device=device) / math.sqrt(D)).bfloat16()
    q, k, v = rn(T, H, D), rn(T, KVH, D), rn(T, KVH, D)
    gq, gk, gv = torch.relu(rn(T, H, D)), torch.relu(rn(T, KVH, D)), rn(T, KVH, D)
    gg = (torch.nn.functional.logsigmoid(torch.randn(T, KVH, D, device=device)) / 16).bfloat16()
    out, gout = torch.empty(T, H, D, dtype=torch.bfloat16, device=device), torch.empty(T, H, D, dtype=torch.bfloat16, device=device)
    n_new = torch.full((S,), chunk, dtype=torch.int32, device=device)
    scan_ws = ops.gla_scan_workspace(S, chunk, H, D, device)
    gla_status = torch.zeros(1, dtype=torch.int32, device=device)
    pin = lambda t: t.cpu().pin_memory()
    host_in = [pin(t) for t in (q, k, v, gq, gk, gv, gg)]
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = d2h = 0

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def prefill_chunk(pos, e2e, trim=True):
        nonlocal h2d, d2h
        plan.plan(n_new)
        meta = MetaAttentionMetadata(
            num_prefills=S, num_prefill_tokens=T, num_decode_tokens=0, slot_mapping=plan.slot_mapping,
            seq_lens=[pos + chunk] * S, seq_lens_tensor=plan.seq_lens, max_prefill_seq_len=pos + chunk,
            max_decode_seq_len=0, context_lens_tensor=plan.context_lens, block_tables=plan.block_tables,
            use_cuda_graph=False, max_query_len=chunk, query_start_loc=plan.query_start_loc)
        for i in range(max(n_swa, n_gla)):
            if i < n_gla:
                if e2e:
                    for dst, src in zip((gq, gk, gv, gg), host_in[3:]):
                        dst.copy_(src, non_blocking=True); h2d += src.numel() * 2
                gla_prefill_scan(gq, gk, gv, gg, gla.cache[i], slot_idx, plan.query_start_loc, plan.context_lens,
                                 status=gla_status, max_query_len=chunk, workspace=scan_ws, out=gout)
                if e2e:
                    host_out.copy_(gout, non_blocking=True); d2h += gout.numel() * 2
            if i < n_swa:
                if e2e:
                    for dst, src in zip((q, k, v), host_in[:3]):
                        dst.copy_(src, non_blocking=True); h2d += src.numel() * 2
                impls[i].forward(None, q, k, v, None, None, None, kv[i], meta, output=out)
                if e2e:
                    host_out.copy_(out, non_blocking=True); d2h += out.numel() * 2
        if trim:
            plan.trim()  # the chunk's look-back window goes back to the ring at once

    def reset_state():
        ops.pool_init(plan.ring, plan.ctrl, plan.seq_lens, plan.block_tables)
        gla.cache.zero_()

    def prefill(e2e, trim_last=True):
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        n_chunks = prompt // chunk
        for c in range(n_chunks):
            prefill_chunk(c * chunk, e2e, trim=trim_last or c + 1 < n_chunks)
        e1.record()
        torch.cuda.synchronize()
        ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3 if e2e else 0.0)
        return max_over_ranks(ms, device)

    # decode step: the same tensors' first S rows are the step's one token per sequence
    q1, k1, v1 = q[:S].contiguous(), k[:S].contiguous(), v[:S].contiguous()
    g1 = [t[:S].reshape(S, t.shape[1], 1, D).contiguous() for t in (gq, gk, gv, gg)]
    out1, gout1 = torch.empty(S, H, D, dtype=torch.bfloat16, device=device), torch.empty(S, H, D, dtype=torch.bfloat16, device=device)
    h1 = [pin(t) for t in (q1, k1, v1, *g1)]
    h_out1 = torch.empty(out1.shape, dtype=out1.dtype).pin_memory()

    def enqueue_decode(e2e):
        nonlocal h2d, d2h
        plan.plan()
        meta = MetaAttentionMetadata(
            num_prefills=0, num_prefill_tokens=0, num_decode_tokens=S, slot_mapping=plan.slot_mapping[:S], seq_lens=None,
            seq_lens_tensor=plan.seq_lens, max_prefill_seq_len=0, max_decode_seq_len=prompt + dsteps,
            context_lens_tensor=None, block_tables=plan.block_tables, use_cuda_graph=False, max_query_len=1,
            max_decode_query_len=1)
        for i in range(max(n_swa, n_gla)):
            if i < n_gla:
                if e2e:
                    for dst, src in zip(g1, h1[3:]):
                        dst.copy_(src, non_blocking=True); h2d += src.numel() * 2
                my_fused_recurrent_gla(*g1, kv_caches=gla.cache[i], slot_idx=slot_idx, out=gout1)
                if e2e:
                    h_out1.copy_(gout1, non_blocking=True); d2h += gout1.numel() * 2
            if i < n_swa:
                if e2e:
                    for dst, src in zip((q1, k1, v1), h1[:3]):
                        dst.copy_(src, non_blocking=True); h2d += src.numel() * 2
                impls[i].forward(None, q1, k1, v1, None, None, None, kv[i], meta, output=out1)
                if e2e:
                    h_out1.copy_(out1, non_blocking=True); d2h += out1.numel() * 2

    def capture_decode(e2e):
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            enqueue_decode(e2e)
            with torch.cuda.graph(g, stream=side):
                enqueue_decode(e2e)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        return g

    def decode(graph, n, sync_each):
        barrier()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(n):
            graph.replay()
            if sync_each:
                torch.cuda.current_stream().synchronize()     # the caller holds the step's outputs on the host
        e1.record()
        torch.cuda.synchronize()
        ms = max(e0.elapsed_time(e1), (time.perf_counter() - t0) * 1e3 if sync_each else 0.0)
        return max_over_ranks(ms, device)

    sampler = ClockSampler(local)
    # ---- warm-up: two chunks (kernel attributes, tensor maps, allocator), then start over ----
    for c in range(2):
        prefill_chunk(c * chunk, False)
    reset_state()
    if rank == 0:
        sampler.start()
    launches0 = instr.launches
    prefill_ms = prefill(False, trim_last=False)     # (the last chunk's trim follows the probe below)
    launches_prefill = instr.launches - launches0 + 1
    # ---- the last chunk's kernels once more, alone, on the state the prefill left (that chunk's look-back
    #      window has not been trimmed yet: every block its queries can see is still resident) ----
    def timed(fn, n=5):
        fn()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / n, device)

    qsl = (torch.arange(S + 1, dtype=torch.int32, device=device) * chunk)
    ctx_t = plan.seq_lens - chunk       # as if the last `chunk` tokens of every sequence were this call's
    probe_status = torch.zeros(1, dtype=torch.int32, device=device)
    attn_ms = timed(lambda: ops.swa_prefill(q, kv[0][0], kv[0][1], plan.block_tables, qsl, ctx_t.contiguous(), chunk,
                                            window_left=WINDOW_LEFT, out=out, status=probe_status)) if n_swa else None
    scan_ms = timed(lambda: ops.gla_scan(gq, gk, gv, gg, gla.cache[0], qsl, slot_idx, out=gout, max_query_len=chunk,
                                         workspace=scan_ws)) if n_gla else None
    chain_ms = timed(lambda: ops.gla_scan(gq, gk, gv, gg, gla.cache[0], qsl, slot_idx, out=gout)) if n_gla else None
    attn_flops = 4.0 * D * H * S * sum(min(prompt - chunk + i, WINDOW_LEFT) + 1 for i in range(chunk))

    plan.trim()
    snap = plan.snapshot()
    resident = [sum(1 for e in row if e >= 0) for row in snap["table"]]
    peak_resident_prefill = (n_blocks - snap["min_free"]) / S
    g_dec = capture_decode(False)          # (two steps of the 512 go into the warm-up and the capture)
    launches0 = instr.launches
    enqueue_decode(False)
    launches_per_decode_step = instr.launches - launches0
    for _ in range(max(args.warmup, 3)):
        g_dec.replay()
    n_dec = max(1, dsteps - 3 - max(args.warmup, 3))
    decode_ms = decode(g_dec, n_dec, False)
    clocks = sampler.stop() if rank == 0 else None
    snap_d = plan.snapshot()
    resident_d = max(sum(1 for e in row if e >= 0) for row in snap_d["table"])

    # ---- end to end: the layers' inputs come from pinned host memory and their outputs go back, per layer ----
    e2e_obj = None
    if not args.no_e2e:
        reset_state()
        h2d = d2h = 0
        e2e_prefill_ms = prefill(True)
        g_e2e = capture_decode(True)
        per_step_in, per_step_out = h2d, d2h
        h2d = d2h = 0
        enqueue_decode(True)
        torch.cuda.synchronize()
        per_step_in, per_step_out = h2d, d2h
        e2e_decode_ms = decode(g_e2e, n_dec, True)
        e2e_obj = {"value": S * world * n_dec / (e2e_decode_ms * 1e-3), "unit": "tokens/s",
                   "h2d_bytes_per_step": per_step_in, "d2h_bytes_per_step": per_step_out,
                   "ms_per_step": e2e_decode_ms / n_dec,
                   "prefill_tokens_per_s": S * world * prompt / (e2e_prefill_ms * 1e-3),
                   "prefill_h2d_bytes_per_chunk": sum(t.numel() * 2 for t in host_in[3:]) * n_gla + sum(t.numel() * 2 for t in host_in[:3]) * n_swa,
                   "prefill_d2h_bytes_per_chunk": out.numel() * 2 * (n_gla + n_swa)}
    status = int(plan.status.item()) | int(gla_status.item()) | int(probe_status.item())
    for impl in impls:
        status |= impl.status()
    if status != 0:
        raise SystemExit(f"rank {rank}: device status {status}; the run is void")
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    tf_peak = float(json.load(open(peaks_path))["bf16_tflops_sustained"]) if os.path.exists(peaks_path) else 1400.0
    attn_tflops = attn_flops / (attn_ms * 1e-3) / 1e12 if attn_ms else None
    ms_per_step = decode_ms / n_dec
    print(json.dumps({
        "metric": "decode tokens/s and cache HBM GB/s (% of 8 TB/s)", "value": S * world * n_dec / (decode_ms * 1e-3),
        "unit": "tokens/s", "n_gpus": world, "steps": n_dec, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16 K/V, f32 GLA state",
        "data": "synthetic",
        "config": {"workload": f"long-context eviction: {S} sequence(s) per GPU, prompt {prompt} in chunks of {chunk} "
                               f"through the block tables, then {dsteps} decode steps; cache path of {n_swa} sliding-window + "
                               f"{n_gla} GLA layers, window_left {WINDOW_LEFT}, block {BLOCK}, 28/4 heads, head_dim 128",
                   "parallelism": f"sequence-sharded x{world}, no collective",
                   "launch": "prefill: host launches, one planner launch per chunk; decode: CUDA graph replay",
                   "l2": "decode at one sequence per GPU is launch-bound (its window, 8 MB per layer, fits L2); the prefill "
                         "kernels are compute-bound"},
        "prefill_tokens_per_s": S * world * prompt / (prefill_ms * 1e-3), "prefill_ms": prefill_ms,
        "prefill_ms_per_chunk": prefill_ms / (prompt // chunk),
        "prefill_attention": {"ms_per_chunk_layer_at_full_window": attn_ms, "useful_tflops": attn_tflops,
                              "frac_of_bf16_sustained": attn_tflops / tf_peak if attn_tflops else None,
                              "peak_tflops": tf_peak},
        "gla_scan": {"ms_per_chunk_layer": scan_ms, "one_chain_per_head_ms": chain_ms,
                     "form": {1: "CUDA cores, one chain per (sequence, head)",
                              2: "tensor cores (tcgen05), one chain per (sequence, head)",
                              3: "tensor cores (tcgen05), runs in two pieces: local pass + full pass",
                              4: "tensor cores (tcgen05), chunk-parallel: local pass, carry, full pass"}[
                         instr._scan_launches((gq, gk, gv, gg, None, qsl), {"workspace": scan_ws, "max_query_len": chunk})]},
        "resident_blocks_per_seq": {"after_prefill": max(resident), "peak_during_prefill": peak_resident_prefill,
                                    "after_decode": resident_d, "window_bound": WINDOW_LEFT // BLOCK + 2,
                                    "whole_history_would_need": (prompt + dsteps) // BLOCK + 1},
        "e2e": e2e_obj, "gpu_launches": launches_prefill + launches_per_decode_step * n_dec,
        "clocks": clocks, "device_status": status}))
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    """The reference's CPU path (oracle port) on the host cores; rank 0 only."""
    if int(os.environ.get("RANK", 0)) != 0:
        return
    sample_seqs = 8
    cores = use_all_host_threads()
    pairs = max(args.swa_layers, args.gla_layers)
    for _ in range(max(args.warmup, 1)):
        cpu_reference_step_seconds(sample_seqs, args.ctx + 1, 1)
    ts = [cpu_reference_step_seconds(sample_seqs, args.ctx + 1, 1) for _ in range(args.steps)]
    t = statistics.mean(ts)
    step_s = t / sample_seqs * args.batch * pairs
    value = args.batch / step_s
    sample = (f"each step: {sample_seqs} sequences x (1 sliding-window layer + 1 GLA layer) at ctx {args.ctx + 1}, "
              f"scaled x{args.batch / sample_seqs:g} sequences x{pairs} layer pairs")
    print(json.dumps({
        "impl": "reference", "metric": "decode tokens/s and cache HBM GB/s (% of 8 TB/s)", "value": value,
        "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 1),
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16 K/V, f32 GLA state", "data": "synthetic",
        "config": {"workload": workload_name(args), "parallelism": "host cores of rank 0"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_head_shard(args):
    """Continuous-batching churn shapes, head-sharded: every rank holds all sequences but only its kv
    heads, decodes its query heads and needs every rank's head outputs afterwards. Times one
    sliding-window layer three ways, on the device, max over ranks: the local kernel alone, kernel +
    NCCL all-gather (+ the copy into head order), and the kernel that stores its rows to the peers
    itself followed by the flag wait (replayed from a CUDA graph, as a serving loop would)."""
    import numpy as np
    import torch
    import torch.distributed as dist
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    rank, world = dist_setup("nccl", device)
    if world < 2:
        raise SystemExit("--head-shard needs at least two ranks (torch.distributed.run, one rank per GPU)")
    from spikingbrain_7b_b200 import ops
    from spikingbrain_7b_b200.head_shard import FusedHeadGather, all_gather_heads, make_hybrid_layout, shard_heads
    # head shards inside a group, sequences across groups (28 heads do not split 8 ways: 8 GPUs run
    # as 4 head shards x 2 sequence groups)
    lay = make_hybrid_layout(args.tp or world)
    tp = lay.tp_size
    qh, kh = shard_heads(H, KVH, tp, lay.tp_rank)
    Hl, kvl = len(qh), len(kh)
    all_lens = np.clip(np.random.default_rng(0).zipf(1.2, size=1024), 128, 65536).astype(np.int64)
    mine = lay.my_sequences(len(all_lens))
    lens_np = all_lens[mine.start:mine.stop]
    B = len(lens_np)
    nblk = (lens_np + BLOCK - 1) // BLOCK
    first = np.maximum(0, lens_np - 1 - WINDOW_LEFT) // BLOCK
    live = nblk - first
    nb = int(live.sum())
    g = torch.Generator().manual_seed(1)
    perm = torch.randperm(nb, generator=g).to(torch.int32)          # a fragmented pool: blocks in random order
    table = torch.full((B, int(nblk.max())), -1, dtype=torch.int32)
    o = 0
    for b in range(B):
        table[b, first[b]:nblk[b]] = perm[o:o + live[b]]
        o += int(live[b])
    table = table.to(device)
    lens = torch.from_numpy(lens_np.astype(np.int32)).to(device)
    n_pools = 3                                                     # layers rotate over pools larger than L2 together
    pools = [torch.randn(2, nb, BLOCK, kvl, D, device=device, dtype=torch.bfloat16) / math.sqrt(D) for _ in range(n_pools)]
    q = (torch.randn(B, Hl, D, device=device) / math.sqrt(D)).bfloat16()
    visible_bytes = float(np.minimum(lens_np, WINDOW_LEFT + 1).sum()) * kvl * D * 2 * 2
    vis = min(table.shape[1] * BLOCK, WINDOW_LEFT + 1)
    split = ops.swa_auto_split(B, vis, device)
    mp = ops.swa_max_pieces(vis, split, B, device)
    ws = ops.swa_workspace(B, Hl, D, mp, device)
    fg = FusedHeadGather(B, H, D, group=lay.tp_group, device=device, timeout_ms=5000)
    out_l = torch.empty(B, Hl, D, dtype=torch.bfloat16, device=device)
    out_g = torch.empty(B, H, D, dtype=torch.bfloat16, device=device)
    kw = dict(window_left=WINDOW_LEFT, workspace=ws, max_pieces=mp, split_chunks=split)

    def local_only(i):
        ops.swa_decode(q, pools[i % n_pools][0], pools[i % n_pools][1], table, lens, out=out_l, **kw)

    def with_nccl(i):
        local_only(i)
        all_gather_heads(out_l, group=lay.tp_group, out=out_g)

    def fused(i):
        return fg.decode(q, pools[i % n_pools][0], pools[i % n_pools][1], table, lens, **kw)

    # parity of the two gathers before anything is timed
    local_only(0)
    want = all_gather_heads(out_l, group=lay.tp_group, out=out_g).clone()      # (a group of one returns its input)
    got = fused(0).clone()
    torch.cuda.synchronize()
    if not torch.equal(got, want) or fg.status.item() != 0:
        raise SystemExit(f"rank {rank}: fused gather differs from the collective (status {fg.status.item()})")
    fused(1)                                                        # an even number of calls before the capture
    n_graph = 2 * n_pools
    side = torch.cuda.Stream(device=device)
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side), torch.cuda.graph(graph, stream=side):
        for i in range(n_graph):
            fused(i)
    torch.cuda.current_stream().wait_stream(side)

    def timed(fn, per_call):
        for i in range(max(args.warmup, 3)):
            fn(i)
        dist.barrier(); torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.steps):
            fn(i)
        e1.record()
        dist.barrier(); torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / args.steps / per_call, device) * 1e3      # microseconds

    t_local = timed(local_only, 1)
    t_nccl = timed(with_nccl, 1)
    t_fused_eager = timed(fused, 1)
    if fg.calls & 1:
        fused(0)               # the graph begins on the first buffer: keep consecutive steps on different ones
    t_fused = timed(lambda i: graph.replay(), n_graph)

    # ---- the GLA layer of the same step: state [B, H/tp, D, D] fp32 per rank, two copies in rotation ----
    gq = torch.relu(torch.randn(B, Hl, D, device=device) / math.sqrt(D)).bfloat16()
    gk = torch.relu(torch.randn(B, kvl, D, device=device) / math.sqrt(D)).bfloat16()
    gv = (torch.randn(B, kvl, D, device=device) / math.sqrt(D)).bfloat16()
    gg = (torch.nn.functional.logsigmoid(torch.randn(B, kvl, D, device=device)) / 16).bfloat16()
    states = [torch.randn(B, Hl, D, D, device=device) * 0.01 for _ in range(2)]
    gla_bytes = 2.0 * B * Hl * D * D * 4

    def gla_local(i):
        ops.gla_step(gq, gk, gv, gg, states[i & 1], out=out_l)

    def gla_nccl(i):
        gla_local(i)
        all_gather_heads(out_l, group=lay.tp_group, out=out_g)

    def gla_fused(i):
        return fg.gla_step(gq, gk, gv, gg, states[i & 1])

    gla_fused(0); gla_fused(1)
    side.wait_stream(torch.cuda.current_stream())
    gla_graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side), torch.cuda.graph(gla_graph, stream=side):
        for i in range(4):
            gla_fused(i)
    torch.cuda.current_stream().wait_stream(side)
    t_gla_local = timed(gla_local, 1)
    t_gla_nccl = timed(gla_nccl, 1)
    t_gla_fused = timed(lambda i: gla_graph.replay(), 4)
    status = fg.status.item()
    fg.close()
    if rank == 0:
        print(json.dumps({
            "metric": "head_sharded_swa_layer_time", "unit": "us", "higher_is_better": False, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "dtype": "bf16", "data": "synthetic",
            "local_kernel_us": round(t_local, 2), "kernel_plus_nccl_all_gather_us": round(t_nccl, 2),
            "fused_gather_graph_us": round(t_fused, 2), "fused_gather_eager_us": round(t_fused_eager, 2),
            "local_kernel_gbs": round(visible_bytes / t_local / 1e3, 1), "status": status,
            "gla_local_kernel_us": round(t_gla_local, 2), "gla_kernel_plus_nccl_all_gather_us": round(t_gla_nccl, 2),
            "gla_fused_gather_graph_us": round(t_gla_fused, 2),
            "gla_local_kernel_gbs": round(gla_bytes / t_gla_local / 1e3, 1),
            "gathered_bytes_per_rank": B * H * D * 2, "whole_job_sequences_per_layer_s": round(
                len(all_lens) / (max(t_fused, 1e-9) * 1e-6)),
            "config": {"workload": f"churn shapes: {len(all_lens)} sequences ({B} per sequence group), ctx Zipf(1.2) "
                                   f"clipped to [128, 65536], window_left {WINDOW_LEFT}, block {BLOCK}, {H}/{KVH} heads "
                                   f"split {tp} ways ({Hl} q / {kvl} kv heads per GPU), head_dim {D}; inputs larger "
                                   f"than L2 ({n_pools} pools of {visible_bytes / 1e6:.0f} MB visible each in rotation)",
                       "parallelism": f"tp{tp} x {lay.n_seq_groups} sequence groups"}}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    a = parse_args()
    if a.head_shard:
        run_head_shard(a)
    elif a.impl == "reference":
        run_reference(a)
    elif a.config == 4:
        run_longctx(a)
    else:
        run_b200(a)
