"""Sharded checkpoint and resume.

The reference can only serialise architecture and strategy (v1 JSON); it has no way to save or restore training
state.  A checkpoint here is a directory:

    meta.json            step, world size, optimizer kind, strategy digest, per-parameter layout, file checksums
    strategy.json        the (mapped) parallel computation graph in the v1 format
    rank<r>.pt           that rank's shard of the fp32 master weights, optimizer moments and RNG state

Each rank writes its own file; rank 0 writes the metadata last, so a directory without ``meta.json`` is an
incomplete checkpoint and is ignored by :func:`latest`.  Files are checksummed and verified on load.
"""
from __future__ import annotations

import hashlib
import json
import os
import re
from typing import Dict, List, Optional

import torch


class CheckpointError(RuntimeError):
    pass


def _sha(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def save(directory: str, executable, step: Optional[int] = None, *, rank: int = 0, world_size: int = 1, strategy=None,
         barrier=None, extra: Optional[dict] = None) -> str:
    if world_size > 1 and barrier is None:
        # without a barrier rank 0 could write the metadata (and its checksum list) before the other ranks' files exist
        raise CheckpointError("save() with world_size > 1 needs a barrier callable (e.g. torch.distributed.barrier)")
    step = executable.step_count if step is None else step
    path = os.path.join(directory, f"step{step:08d}")
    os.makedirs(path, exist_ok=True)
    sd = {k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in executable.state_dict().items()}
    sd["rng_cpu"] = torch.get_rng_state()
    layout = {}
    if hasattr(executable, "param_nodes"):  # arena executors; the host executor keeps its parameters by name
        layout = {name: {"offset": executable.param_offsets[nid][0], "numel": executable.param_offsets[nid][1],
                         "shape": list(executable.local_weight_shape(nid))}
                  for nid, name in ((n, executable.nodes[n]["name"] or f"weight{n}") for n in executable.param_nodes)}
    sd["layout"] = layout
    fn = os.path.join(path, f"rank{rank}.pt")
    tmp = fn + ".tmp"
    torch.save(sd, tmp)
    os.replace(tmp, fn)
    if barrier is not None:
        barrier()
    if rank == 0:
        if strategy is not None:
            with open(os.path.join(path, "strategy.json"), "w") as f:
                f.write(strategy.to_v1_string(parallel=True))
        files = sorted(x for x in os.listdir(path) if x.startswith("rank") and x.endswith(".pt"))
        meta = {"step": int(step), "world_size": world_size, "optimizer": executable.cfg.optimizer.kind,
                "compute_dtype": executable.cfg.compute_dtype, "files": {x: _sha(os.path.join(path, x)) for x in files},
                "extra": extra or {}}
        tmp = os.path.join(path, "meta.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f, indent=1)
        os.replace(tmp, os.path.join(path, "meta.json"))
    if barrier is not None:
        barrier()
    return path


def latest(directory: str) -> Optional[str]:
    """Newest complete checkpoint under `directory` (None if there is none)."""
    if not os.path.isdir(directory):
        return None
    best = None
    for d in sorted(os.listdir(directory)):
        if re.fullmatch(r"step\d{8}", d) and os.path.exists(os.path.join(directory, d, "meta.json")):
            best = os.path.join(directory, d)
    return best


def load(path: str, executable, *, rank: int = 0, verify: bool = True) -> dict:
    meta_fn = os.path.join(path, "meta.json")
    if not os.path.exists(meta_fn):
        raise CheckpointError(f"{path} has no meta.json (incomplete checkpoint)")
    with open(meta_fn) as f:
        meta = json.load(f)
    fn = os.path.join(path, f"rank{rank}.pt")
    if not os.path.exists(fn):
        raise CheckpointError(f"{fn} is missing: the checkpoint was written by {meta['world_size']} ranks")
    if verify:
        want = meta["files"].get(os.path.basename(fn))
        if want is None:
            raise CheckpointError(f"{fn} has no recorded checksum in meta.json (written after the metadata?)")
        if _sha(fn) != want:
            raise CheckpointError(f"{fn} does not match its recorded checksum (corrupt file)")
    try:
        sd = torch.load(fn, map_location="cpu", weights_only=False)
    except Exception as e:
        raise CheckpointError(f"{fn} cannot be read: {e}") from e
    if ("master" in sd) != hasattr(executable, "master"):
        raise CheckpointError("the checkpoint was written by another kind of executor (arena / host); use load_resharded")
    if "master" in sd and sd["master"].numel() != executable.master.numel():
        raise CheckpointError("parameter arena size differs: the checkpoint belongs to another model or strategy "
                              "(use load_resharded to change the strategy)")
    executable.load_state_dict(sd)
    if "rng_cpu" in sd:
        torch.set_rng_state(sd["rng_cpu"])
    return meta


def gather_full_parameters(path: str) -> Dict[str, torch.Tensor]:
    """All parameters of a single-rank (or replicated) checkpoint by name, as fp32 tensors."""
    sd = torch.load(os.path.join(path, "rank0.pt"), map_location="cpu", weights_only=False)
    out = {}
    if "params" in sd:  # written by the host executor: parameters by name
        return {k: v.to(torch.float32) for k, v in sd["params"].items()}
    for name, l in sd["layout"].items():
        out[name] = sd["master"][l["offset"]:l["offset"] + l["numel"]].view(l["shape"]).clone()
    # sparsely updated embedding tables are stored whole, under "table.<name>", by the rank that owns them
    for fn in sorted(x for x in os.listdir(path) if re.fullmatch(r"rank\d+\.pt", x)):
        other = sd if fn == "rank0.pt" else torch.load(os.path.join(path, fn), map_location="cpu", weights_only=False)
        for k, v in other.items():
            if isinstance(k, str) and k.startswith("table."):
                out[k[len("table."):]] = v.to(torch.float32)
    return out


def load_resharded(path: str, executable) -> dict:
    """Restore parameters by *name* from a checkpoint whose weights are whole (single rank or data parallel) into
    an executable with any strategy: each weight is re-sliced with the executable's own sharding rule.
    Optimizer moments restart from zero."""
    full = gather_full_parameters(path)
    for nid in executable.param_nodes:
        name = executable.nodes[nid]["name"] or f"weight{nid}"
        if name not in full:
            raise CheckpointError(f"parameter {name} is not in the checkpoint")
        o, n = executable.param_offsets[nid]
        shard = executable.shard_weight(nid, full[name].view(list(executable.nodes[nid]["outputs"][0][1].sizes)))
        executable.master[o:o + n].copy_(shard.reshape(-1))
    for nid, t in getattr(executable, "sparse_tables", {}).items():
        name = executable.nodes[nid]["name"] or str(nid)
        if t is not None:
            if name not in full:
                raise CheckpointError(f"embedding table {name} is not in the checkpoint")
            t.copy_(full[name].view(t.shape))
    if executable.shadow is not None:
        executable.shadow.copy_(executable.master)
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    executable.step_count = int(meta["step"])
    return meta
