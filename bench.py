#!/usr/bin/env python
"""Headline benchmark: training throughput (samples/s) of the large lib/models-style Transformer
(24 decoder-only layers, d_model 2048, 16 heads, FFN 8192, vocab 32000, seq 1024, global batch 32,
bf16 compute with fp32 master weights, Adam) on N GPUs of one node.

  python bench.py --gpus 1 --steps 10 --warmup 3
  python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
      bench.py --gpus N --steps K --warmup W

Prints one JSON line on rank 0.  `value` is device-timed (CUDA events, max over ranks) with the batch
already on the device; `e2e` times the public API (`CompiledModel.train_step`) including the
host->device copy of every step's batch from pinned memory and the device->host read of the loss.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

MODEL_CONFIGS = {
    "transformer_large": ("transformer_lm", {"num_features": 2048, "sequence_length": 1024, "batch_size": 32,
                                             "dim_feedforward": 8192, "num_heads": 16, "num_decoder_layers": 24,
                                             "dropout": 0.1, "vocab_size": 32000, "init_std": 0.02}),
    "transformer_small": ("transformer_lm", {"num_features": 512, "sequence_length": 256, "batch_size": 8,
                                             "dim_feedforward": 2048, "num_heads": 8, "num_decoder_layers": 2,
                                             "dropout": 0.1, "vocab_size": 4096}),
    "bert_base": ("bert", {"token_ids": True, "batch_size": 64, "sequence_length": 512, "vocab_size": 30528}),
    "inception_v3": ("inception_v3", {"batch_size": 256, "num_classes": 1000}),
    "dlrm": ("dlrm", {"batch_size": 4096, "embedding_dim": 64, "embedding_bag_size": 1, "embedding_size": [1000000] * 8,
                      "dense_arch_layer_sizes": [13, 512, 256, 64], "over_arch_layer_sizes": [512, 512, 256, 1],
                      "arch_interaction_op": "DOT", "final_activation": "SIGMOID", "embedding_data_type": "FLOAT",
                      "embedding_init_range": 0.01}),
}
# optimizer and loss per model, as the benchmark configurations name them
TRAINING = {
    "transformer_large": ("adam", 1e-4, 0.0, "sparse_categorical_crossentropy"),
    "transformer_small": ("adam", 1e-4, 0.0, "sparse_categorical_crossentropy"),
    "bert_base": ("adam", 1e-4, 0.0, "sparse_categorical_crossentropy"),
    "inception_v3": ("sgd", 0.01, 0.9, "sparse_categorical_crossentropy"),
    "dlrm": ("sgd", 0.01, 0.0, "mean_squared_error_avg_reduce"),
}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.proc = None
        self.lines = []
        self.gpu_index = gpu_index
        self.nvml = None       # (module, device handle) when NVML can be read in-process
        self.samples = []      # (sm MHz, max MHz, reason bitmask) from NVML
        self._stop = False

    def _nvml_open(self):
        import pynvml
        pynvml.nvmlInit()
        h = None
        try:  # the CUDA device's own UUID, so that device ordering cannot pick another GPU
            import torch
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            h = None
        if h is None:
            h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)
        pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)  # fails here rather than in the thread
        return pynvml, h

    def _nvml_sample(self):
        nv, h = self.nvml
        try:
            sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
            self.samples.append((float(sm), float(mx), int(get(h))))
        except Exception:
            pass

    def _nvml_loop(self):
        # read-only queries; every 5 ms for the first second (a timed region can be a few milliseconds), then every 100 ms
        n = 0
        while not self._stop:
            self._nvml_sample()
            n += 1
            time.sleep(0.005 if n < 200 else 0.1)

    def start(self):
        try:
            self.nvml = self._nvml_open()
            self.thread = threading.Thread(target=self._nvml_loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                                          "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self._nvml_sample()  # at least one reading taken while the last timed kernels are still in flight
            self._stop = True
            self.thread.join(timeout=2)
            sm = sorted(x[0] for x in self.samples)
            mask = 0
            for x in self.samples:
                mask |= x[2]
            names = (("sw_power_cap", 0x4), ("hw_slowdown", 0x8), ("sw_thermal_slowdown", 0x20), ("hw_thermal_slowdown", 0x40))
            return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max((x[1] for x in self.samples), default=None),
                    "reasons": sorted(n for n, bit in names if mask & bit), "samples": len(sm), "source": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# how each model's timed steps relate to the 126 MB L2 (timing rule: inputs larger than L2, or a flush between steps)
L2_NOTE = {
    "transformer_large": "activations and weights per step (>100 GB) exceed the 126 MB L2; no flush needed",
    "transformer_small": "weights, optimizer state and activations per step (>1 GB) exceed the 126 MB L2; no flush needed",
    "bert_base": "activations and weights per step (>10 GB) exceed the 126 MB L2; no flush needed",
    "inception_v3": "activations per step (>20 GB) exceed the 126 MB L2; no flush needed",
    "dlrm": "2 GB of embedding tables, rows drawn at random: every step's lookups miss L2; the MLP working set (a few MB) stays resident, as it does in training",
}


def reference_arm(args):
    # The reference is C++/CMake with no Python project at its root; the one offline pip install that is
    # allowed fails before any build starts (no setup.py / pyproject.toml; its legacy bindings need the
    # absent cmake_build_extension package and a Legion runtime).  Nothing of it can be run here.
    print(json.dumps({"impl": "reference", "unavailable":
                      "pip install of the reference tree fails offline: no setup.py/pyproject.toml at its root; "
                      "bindings/python/old needs cmake_build_extension + Legion/Realm, not in the wheelhouse"}))
    return 0


def torch_arm(args):
    """Library baseline (B1): the same model, data and step contents in stock PyTorch -- cuBLAS / cuDNN / the library
    attention kernel under bf16 autocast with fp32 parameters and torch.optim, one process per GPU with gradients
    averaged across ranks (DistributedDataParallel for the module-based Transformer, one flat all-reduce for the
    graph-interpreted models).  None of this repository's kernels or executors are on this path."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    model_name, mcfg = MODEL_CONFIGS[args.model]
    mcfg = dict(mcfg)
    opt_kind, lr, momentum, loss_kind = TRAINING[args.model]
    global_batch, seq = mcfg["batch_size"], mcfg.get("sequence_length", 1)
    if global_batch % world:
        raise SystemExit(f"global batch {global_batch} does not divide over {world} ranks")
    local_batch = global_batch // world
    warmup = max(args.warmup, 3)
    gen = torch.Generator().manual_seed(1234 + rank)
    try:
        if model_name == "transformer_lm":
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import torch_models
            torch.manual_seed(0)
            net = torch_models.build_transformer_lm(mcfg).cuda()
            params = list(net.parameters())
            mod = torch.nn.parallel.DistributedDataParallel(net, device_ids=[local_rank], gradient_as_bucket_view=True) if world > 1 else net
            vocab = mcfg["vocab_size"]
            host = [(torch.randint(0, vocab, (local_batch, seq), generator=gen, dtype=torch.int64).pin_memory(),
                     torch.randint(0, vocab, (local_batch, seq), generator=gen, dtype=torch.int64).pin_memory()) for _ in range(4)]

            def fwd_bwd(ids, lab):
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = mod(ids, lab)
                loss.backward()
                return loss
        else:
            from flexflow_train_b200 import _ffcore as core
            from flexflow_train_b200.bin.run_model import synthetic_batch
            from flexflow_train_b200.runtime.torch_oracle import TorchOracle
            g = core.build_model(model_name, dict(mcfg, batch_size=local_batch))
            orc = TorchOracle(g, loss=loss_kind, seed=0, device="cuda", dropout=True)
            orc.use_sdpa = True
            params = list(orc.params.values())
            channels_last = model_name == "inception_v3"
            if channels_last:  # what a PyTorch user does for convolution networks on tensor cores
                for prm in params:
                    if prm.dim() == 4:
                        prm.data = prm.data.contiguous(memory_format=torch.channels_last)

            class _Shape:  # the batch generator only needs the loss value of the graph
                loss_value = orc.loss_value
                graph = g
            host = [synthetic_batch(g, _Shape, loss_kind, seed=1234 + 17 * rank + i) for i in range(4)]
            if "vocab_size" in mcfg:
                for ins, lab in host:
                    lab.copy_(torch.randint(0, mcfg["vocab_size"], lab.shape, generator=gen, dtype=lab.dtype))

            def fwd_bwd(ins, lab):
                if channels_last:
                    ins = {k: (v.contiguous(memory_format=torch.channels_last) if v.dim() == 4 else v) for k, v in ins.items()}
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    pred = orc.forward(ins)
                loss = orc.loss(pred.float(), lab).mean()
                loss.backward()
                if world > 1:  # data parallel: one flat all-reduce of the gradients
                    grads = [prm.grad for prm in params if prm.grad is not None]
                    flat = torch._utils._flatten_dense_tensors(grads)
                    dist.all_reduce(flat)
                    flat.div_(world)
                    for gr, fl in zip(grads, torch._utils._unflatten_dense_tensors(flat, grads)):
                        gr.copy_(fl)
                return loss
        opt = torch.optim.Adam(params, lr=lr, fused=True) if opt_kind == "adam" else torch.optim.SGD(params, lr=lr, momentum=momentum)

        def to_dev(batch):
            a, b_ = batch
            if isinstance(a, dict):
                return {k: v.cuda(non_blocking=True) for k, v in a.items()}, b_.cuda(non_blocking=True)
            return a.cuda(non_blocking=True), b_.cuda(non_blocking=True)

        def step(batch):
            opt.zero_grad(set_to_none=True)
            loss = fwd_bwd(*batch)
            opt.step()
            return loss

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        dev = [to_dev(hb) for hb in host]
        for i in range(warmup):
            step(dev[i % 4])
        barrier()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            step(dev[i % 4])
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / args.steps
        clocks = sampler.stop() if rank == 0 else None
        # end to end: pinned host batch -> device and loss -> host every step
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            loss = step(to_dev(host[i % 4]))
            float(loss)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
        h2d = sum(t.numel() * t.element_size() for t in (list(host[0][0].values()) if isinstance(host[0][0], dict) else [host[0][0]])) + \
            host[0][1].numel() * host[0][1].element_size()
    except torch.OutOfMemoryError as e:
        print(json.dumps({"impl": "torch", "unavailable": f"out of memory on this config: {str(e)[:120]}"}))
        return 0
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        print(json.dumps({"metric": "train samples/s (searched strategy)", "value": global_batch / (ms / 1e3), "unit": "samples/s",
                          "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "strong", "vs_baseline": None, "dtype": "bf16 autocast", "data": "synthetic", "impl": "torch",
                          "config": {"model": args.model, "global_batch": global_batch, "seq_len": seq,
                                     "parallelism": f"ddp{world}" if world > 1 else "single", "optimizer": opt_kind, "lr": lr},
                          "clocks": clocks,
                          "e2e": {"value": global_batch / (e2e_ms / 1e3), "unit": "samples/s", "ms_per_step": e2e_ms,
                                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
                          "gpu_launches": 0, "final_loss": float(loss)}))
    if world > 1:
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="transformer_large", choices=sorted(MODEL_CONFIGS))
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--strategy", default="search", help="search | dp | tp | dp<a>xtp<b> (device mesh) | tables (model-parallel embedding tables under a data-parallel model) | <path to strategy json>")
    ap.add_argument("--search-budget", type=int, default=10, help="Unity search budget on top of the scored templates (0 = templates only)")
    ap.add_argument("--search-time-limit", type=float, default=30.0)
    ap.add_argument("--global-batch", type=int, default=None, help="override the model configuration's global batch (experiments; the "
                    "headline configuration is the default)")
    ap.add_argument("--timeline", action="store_true",
                    help="after the timed runs, print rank 0's per-phase and per-bucket timeline of two eager steps (stderr)")
    ap.add_argument("--no-fused-collectives", action="store_true",
                    help="tensor-parallel collectives through NCCL instead of inside the GEMM kernels (baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.impl == "torch":
        return torch_arm(args)
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist
    from flexflow_train_b200 import api
    from flexflow_train_b200.ops import kernels as K
    from flexflow_train_b200.runtime.executor import OptimizerConfig

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    dctx = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from flexflow_train_b200.parallel.context import DistContext
        dctx = DistContext(rank, world, local_rank)

    model_name, mcfg = MODEL_CONFIGS[args.model]
    mcfg = dict(mcfg)
    if args.global_batch:
        mcfg["batch_size"] = args.global_batch
    global_batch, seq = mcfg["batch_size"], mcfg.get("sequence_length", 1)
    opt_kind, lr, momentum, loss_kind = TRAINING[args.model]
    ffcfg = api.FFConfig(batch_size=global_batch, compute_dtype="bf16", use_cuda_graph=not args.no_cuda_graph, seed=0,
                         fuse_collectives=not args.no_fused_collectives, search_budget=args.search_budget,
                         search_time_limit_s=args.search_time_limit,
                         search_algorithm={"search": "unity", "dp": "data_parallel", "tp": "tensor_parallel", "tables": "table_parallel"}.get(
                             args.strategy, args.strategy if "xtp" in args.strategy else "unity"),
                         import_strategy_file=args.strategy if os.path.exists(args.strategy) else None)
    model = api.compile(model_name, mcfg, config=ffcfg, optimizer=OptimizerConfig(kind=opt_kind, lr=lr, momentum=momentum),
                        loss=loss_kind, dist=dctx)
    ex = model.executable
    vocab = mcfg.get("vocab_size", 0)
    # every rank is handed the global batch (token ids are tiny); the strategy's Repartition keeps the local slice
    local_batch = global_batch

    # synthetic data of the named shape: token ids uniform over the vocabulary, next-token labels
    gen = torch.Generator().manual_seed(1234)
    n_host = 4
    if model_name == "bert":
        host_batches = [({"input_ids": torch.randint(0, 30522, (local_batch, seq, 1), generator=gen, dtype=torch.int32).pin_memory(),
                          "position_ids": torch.arange(seq, dtype=torch.int32).repeat(local_batch, 1).reshape(local_batch, seq, 1).pin_memory()},
                         torch.where(torch.rand(local_batch, seq, generator=gen) < 0.15,
                                     torch.randint(0, 30522, (local_batch, seq), generator=gen), torch.tensor(-1)).to(torch.int32).pin_memory())
                        for _ in range(n_host)]
    elif model_name == "transformer_lm":
        host_batches = [({"input_ids": torch.randint(0, vocab, (local_batch, seq, 1), generator=gen, dtype=torch.int32).pin_memory()},
                         torch.randint(0, vocab, (local_batch, seq), generator=gen, dtype=torch.int32).pin_memory())
                        for _ in range(n_host)]
    else:  # images / dense + sparse features drawn as the config names them, shapes from the graph's inputs
        from flexflow_train_b200.bin.run_model import synthetic_batch
        host_batches = [synthetic_batch(model.graph, ex, loss_kind, seed=1234 + i) for i in range(n_host)]
        if model_name == "dlrm":  # binary labels
            host_batches = [(i, (l > 0.5).to(l.dtype).pin_memory()) for i, l in host_batches]
    # Inputs that the strategy splits over the sample dimension are handed to each rank as its own piece (every rank
    # draws the same global batch from the same seed and keeps its rows), so the host-to-device traffic per rank shrinks
    # with the number of ranks; anything else (an input a tensor-parallel plan replicates) is passed whole.
    direct = set(getattr(ex, "direct_inputs", {}))
    if world > 1 and direct:
        # the sample dimension is cut over the data-parallel axis: all ranks on a one-axis plan, the rows of the mesh otherwise
        grp = next(iter(ex.direct_inputs.values())).gctx
        lb = global_batch // grp.world_size

        def rows(t):
            return t[grp.rank * lb:(grp.rank + 1) * lb].contiguous().pin_memory()
        host_batches = [({k: (rows(v) if k in direct else v) for k, v in i.items()}, rows(l.reshape(global_batch, -1))) for i, l in host_batches]
    dev_batches = [({k: v.cuda() for k, v in i.items()}, l.cuda()) for i, l in host_batches]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed: batch resident on the device
    for i in range(args.warmup):
        ex.train_step(*dev_batches[i % n_host])
    barrier()
    l0 = K.launch_count()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        ex.train_step(*dev_batches[i % n_host])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop() if rank == 0 else None
    launches = K.launch_count() - l0
    if ex.cfg.use_cuda_graph:
        launches = getattr(ex, "launches_per_step", 0) * args.steps + launches
    final_loss = ex.mean_loss()

    # ---- end to end through the public API: pinned host batch -> device, loss -> host, every step
    for i in range(2):
        model.train_step(*host_batches[i % n_host])
    barrier()
    t0 = time.perf_counter()
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e2.record()
    for i in range(args.steps):
        model.train_step(*host_batches[i % n_host])
    e3.record()
    barrier()
    e2e_ms = max(e2.elapsed_time(e3), (time.perf_counter() - t0) * 1e3) / args.steps
    h2d, d2h = model.h2d_bytes_last_step, model.d2h_bytes_last_step

    if args.timeline and hasattr(ex, "enable_timeline"):
        # every rank runs the same two eager steps (collectives inside); rank 0 reports
        was = ex.cfg.use_cuda_graph
        ex.cfg.use_cuda_graph = False
        ex.enable_timeline()
        for i in range(2):
            ex.train_step(*dev_batches[i % n_host])
        tl = ex.timeline()
        ex.cfg.use_cuda_graph = was
        if rank == 0:
            print(json.dumps({"timeline_ms": tl}), file=sys.stderr)
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    if rank == 0:
        value = global_batch / (ms / 1e3)
        out = {
            "metric": "train samples/s (searched strategy)", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {"model": args.model, "global_batch": global_batch, "seq_len": seq,
                       "parallelism": getattr(ex, "parallelism", "single"),
                       **({"layers": mcfg.get("num_decoder_layers", mcfg.get("num_encoder_layers", 12)),
                           "d_model": mcfg.get("num_features", mcfg.get("hidden_size", 768))}
                          if model_name in ("transformer_lm", "transformer", "bert") else {}),
                       "optimizer": opt_kind, "lr": lr,
                       "l2": L2_NOTE[args.model],
                       "cuda_graph": bool(ex.cfg.use_cuda_graph), "tokens_per_s": value * seq,
                       "fused_collective_gemms": len(getattr(ex, "fused_in", [])) + len(getattr(ex, "fused_out", []))},
            "clocks": clocks,
            "e2e": {"value": global_batch / (e2e_ms / 1e3), "unit": "samples/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
            "gpu_launches": int(launches), "final_loss": final_loss,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
