"""Checkpoints of distributed runs: ``ckpt-%08d`` directories, save / restore, rotation.

Directory layout and ``checkpoint.json`` fields follow the reference
(src/rwkv7m/distributed/checkpoint.py:34-126,208-302).  Its two backends map
onto this framework as follows: ``single`` (alias ``flax``) lets rank 0 write
the complete train state after gathering any sharded Adam moments; ``sharded``
(alias ``orbax``) lets every rank write its own optimizer shard and runtime
state next to rank 0's model files; a restore may use another world size.
"""

from __future__ import annotations

import json
import shutil
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist
from safetensors.torch import load_file, save_file

from ..config import model_config_from_dict, model_config_to_dict
from ..io.checkpoint import (
    CHECKPOINT_JSON,
    MODEL_SAFETENSORS,
    RUNTIME_STATE_FILE,
    TRAIN_STATE_FILE,
    load_train_checkpoint,
    load_train_runtime_state,
    safetensors_file_is_whole,
    save_runtime_state,
    save_train_checkpoint,
    write_json_atomic,
)
from ..io.names import from_portable, to_portable
from ..io.safetensors_io import save_model_safetensors

TP_SHARD_FILE = "tp_state.rank{rank:05d}.safetensors"
BACKEND_ALIASES = {"flax": "single", "single": "single", "orbax": "sharded", "sharded": "sharded"}


@dataclass(frozen=True)
class DistributedCheckpointPayload:
    config: object
    metadata: dict
    start_step: int
    dataset_position: dict | None


def normalize_backend(name: str) -> str:
    if name not in BACKEND_ALIASES:
        raise ValueError(f"checkpoint backend must be one of {sorted(BACKEND_ALIASES)}")
    return BACKEND_ALIASES[name]


def checkpoint_path(output_dir, step) -> Path:
    return Path(output_dir) / f"ckpt-{int(step):08d}"


def list_checkpoint_dirs(output_dir) -> list:
    output_dir = Path(output_dir)
    if not output_dir.exists():
        return []
    found = []
    for path in output_dir.iterdir():
        if path.is_dir() and path.name.startswith("ckpt-"):
            tail = path.name[len("ckpt-"):]
            if tail.isdigit():
                found.append((int(tail), path))
    return [p for _, p in sorted(found)]


def checkpoint_is_complete(checkpoint_dir) -> bool:
    """True when the directory holds everything a restore reads: a parseable ``checkpoint.json`` (written last), the model
    file, and the state files of its backend (one train-state file, or every rank's shard; per-rank runtime state: all ranks'
    or none), each as long as its own header says (a file cut short by a crash fails without a tensor being read)."""
    checkpoint_dir = Path(checkpoint_dir)
    try:
        with open(checkpoint_dir / CHECKPOINT_JSON, "r", encoding="utf-8") as f:
            payload = json.load(f)
    except (OSError, ValueError):
        return False
    needed = [MODEL_SAFETENSORS]
    if payload.get("backend", "single") == "sharded" and payload.get("layout") == "tensor_parallel":
        needed += [TP_SHARD_FILE.format(rank=r) for r in range(int(payload.get("model_parallel", 1)))]
    elif payload.get("backend", "single") == "sharded":
        needed += [TRAIN_STATE_FILE] + [f"optimizer_shard.rank{r:05d}.safetensors" for r in range(int(payload.get("world_size", 1)))]
    else:
        needed.append(TRAIN_STATE_FILE)
    for r in range(int(payload.get("world_size", 1))):     # carried runtime state, where the run saved one per rank
        if (checkpoint_dir / f"runtime_state.rank{r:05d}.safetensors").exists():
            needed += [f"runtime_state.rank{q:05d}.safetensors" for q in range(int(payload.get("world_size", 1)))]
            break
    return all(safetensors_file_is_whole(checkpoint_dir / name) for name in needed)


def latest_complete_checkpoint(output_dir):
    """The newest ``ckpt-%08d`` directory under ``output_dir`` that a restore can use, or None: what ``--resume auto``
    picks, so that a job restarted after a crash in the middle of a save falls back to the checkpoint before it."""
    if output_dir is None:
        return None
    for path in reversed(list_checkpoint_dirs(output_dir)):
        if checkpoint_is_complete(path):
            return path
    return None


def load_distributed_checkpoint_raw_metadata(checkpoint_dir):
    with open(Path(checkpoint_dir) / CHECKPOINT_JSON, "r", encoding="utf-8") as f:
        payload = json.load(f)
    return model_config_from_dict(payload["config"]), payload


def load_distributed_checkpoint_metadata(checkpoint_dir) -> DistributedCheckpointPayload:
    config, payload = load_distributed_checkpoint_raw_metadata(checkpoint_dir)
    return DistributedCheckpointPayload(config, payload, int(payload.get("step", 0)), payload.get("dataset_position"))


def _world(process_info):
    return int(process_info["process_index"]), int(process_info["process_count"])


def _barrier(process_info):
    if process_info["process_count"] > 1 and dist.is_initialized():
        dist.barrier()


def _moment_shard(train_state):
    """(exp_avg, exp_avg_sq, begin, end) of this rank, or None when moments are replicated."""
    fused = train_state.extras.get("fused_optimizer")
    if fused is None:
        return None
    return fused.exp_avg, fused.exp_avg_sq, fused.begin, fused.end


def _sync_masters(train_state):
    """The fused data-parallel step keeps the fp32 master value of a bulk weight only on its owner: refresh every
    rank's copy before the parameters are read for a checkpoint (collective, no-op otherwise)."""
    fused = train_state.extras.get("fused_optimizer")
    if fused is not None and hasattr(fused, "gather_master"):
        fused.gather_master()


def _gather_moments_into_optimizer(train_state, process_info):
    """Materialise full Adam moments on the optimizer object (every rank) from the per-rank shards."""
    shard = _moment_shard(train_state)
    if shard is None:
        return False
    m, v, begin, end = shard
    opt = train_state.optimizer
    total = opt.flat.master.numel()
    full_m = torch.empty(total, dtype=m.dtype, device=m.device)
    full_v = torch.empty_like(full_m)
    dist.all_gather_into_tensor(full_m, m)
    dist.all_gather_into_tensor(full_v, v)
    opt.exp_avg, opt.exp_avg_sq = full_m, full_v
    return True


def save_data_parallel_checkpoint(*args, **kwargs):
    """Two call forms.  ``(checkpoint_dir, train_state, config, process_info, *, backend=..., ...)`` writes into the
    directory given.  ``(output_dir, step, dist_objects, config, process_info, ...)`` is the reference's
    (src/rwkv7m/distributed/checkpoint.py:208-302): the directory is ``output_dir/ckpt-%08d``, the train state is taken
    from the placed objects, and ``output_dir=None`` saves nothing."""
    if len(args) >= 2 and isinstance(args[1], int) and not isinstance(args[1], bool):
        output_dir, step, objects = args[0], args[1], args[2]
        if output_dir is None:
            return None
        train_state = getattr(objects, "train_state", objects)
        return _save_checkpoint_dir(checkpoint_path(output_dir, step), train_state, *args[3:], **kwargs)
    return _save_checkpoint_dir(*args, **kwargs)


def _save_checkpoint_dir(checkpoint_dir, train_state, config, process_info, *, backend="single",
                         rng_key=None, dataset_position=None, metadata=None, runtime_state=None):
    backend = normalize_backend(backend)
    rank, world = _world(process_info)
    checkpoint_dir = Path(checkpoint_dir)
    tp = train_state.extras.get("tp")
    if tp is not None and backend == "sharded":
        return _save_tensor_parallel_shards(checkpoint_dir, train_state, config, process_info, tp, rng_key=rng_key,
                                            dataset_position=dataset_position, metadata=metadata,
                                            runtime_state=runtime_state)
    if tp is not None:
        # tensor-parallel shards are gathered into full tensors: the files are those of an un-sharded run
        with tp.materialized(train_state):
            if rank == 0:
                save_train_checkpoint(checkpoint_dir, train_state, config, rng_key=rng_key,
                                      dataset_position=dataset_position, metadata=metadata, runtime_state=None)
                _patch_json(checkpoint_dir, {"backend": "single", "world_size": world, "model_parallel": tp.world})
        if runtime_state is not None:   # recurrent state holds this rank's heads: one file per rank
            if rank != 0:
                checkpoint_dir.mkdir(parents=True, exist_ok=True)
            save_runtime_state(checkpoint_dir / f"runtime_state.rank{rank:05d}.safetensors", runtime_state)
        _barrier(process_info)
        return checkpoint_dir
    zero3 = train_state.extras.get("zero3")
    if zero3 is not None:
        # parameters and moments are sharded piece by piece: gather them into the replicated layout for the writer
        if backend != "single":
            raise ValueError("a ZeRO-3 train state is saved with the 'single' checkpoint backend")
        with zero3.materialized():
            if rank == 0:
                save_train_checkpoint(checkpoint_dir, train_state, config, rng_key=rng_key,
                                      dataset_position=dataset_position, metadata=metadata, runtime_state=runtime_state)
                _patch_json(checkpoint_dir, {"backend": "single", "world_size": world})
        _barrier(process_info)
        return checkpoint_dir
    if world > 1:
        _sync_masters(train_state)
    if backend == "single":
        gathered = _gather_moments_into_optimizer(train_state, process_info) if world > 1 else False
        if rank == 0:
            save_train_checkpoint(checkpoint_dir, train_state, config, rng_key=rng_key,
                                  dataset_position=dataset_position, metadata=metadata, runtime_state=runtime_state)
            _patch_json(checkpoint_dir, {"backend": "single", "world_size": world})
        if gathered:
            train_state.optimizer.exp_avg = train_state.optimizer.exp_avg_sq = None
        _barrier(process_info)
        return checkpoint_dir
    # sharded: every rank writes its part
    if rank == 0:
        checkpoint_dir.mkdir(parents=True, exist_ok=True)
    _barrier(process_info)
    shard = _moment_shard(train_state)
    opt = train_state.optimizer
    if shard is None:
        total = opt.flat.master.numel()
        per = total // world if total % world == 0 else total
        begin, end = (rank * per, (rank + 1) * per) if per != total else (0, total if rank == 0 else 0)
        m, v = opt.exp_avg[begin:end], opt.exp_avg_sq[begin:end]
    else:
        m, v, begin, end = shard
    save_file(
        {"exp_avg": m.detach().contiguous().cpu(), "exp_avg_sq": v.detach().contiguous().cpu(),
         "range": torch.tensor([begin, end], dtype=torch.int64)},
        str(checkpoint_dir / f"optimizer_shard.rank{rank:05d}.safetensors"),
    )
    if runtime_state is not None:
        save_runtime_state(checkpoint_dir / f"runtime_state.rank{rank:05d}.safetensors", runtime_state)
    if rank == 0:
        tensors = {f"model/{k}": v for k, v in to_portable(train_state.model).items()}
        tensors["optimizer/count"] = torch.tensor([opt.count], dtype=torch.int64)
        save_file(tensors, str(checkpoint_dir / TRAIN_STATE_FILE))
        save_model_safetensors(checkpoint_dir / MODEL_SAFETENSORS, train_state.model, config,
                               metadata={"checkpoint_step": int(train_state.step), **(metadata or {})})
        payload = {
            "format": "rwkv7m_train_checkpoint", "format_version": 1, "backend": "sharded", "world_size": world,
            "step": int(train_state.step), "config": model_config_to_dict(config),
            "rng_key": None if rng_key is None else [int(x) for x in torch.as_tensor(rng_key).reshape(-1).tolist()],
            "dataset_position": dataset_position, "metadata": metadata or {},
        }
    _barrier(process_info)      # every rank's shard is on disk before the file that marks the checkpoint as finished
    if rank == 0:
        write_json_atomic(checkpoint_dir / CHECKPOINT_JSON, payload)
    _barrier(process_info)
    return checkpoint_dir


def _save_tensor_parallel_shards(checkpoint_dir, train_state, config, process_info, tp, *, rng_key, dataset_position,
                                 metadata, runtime_state):
    """Sharded backend for a tensor-parallel train state: every rank of one model-parallel group writes its own flat fp32
    master buffer and both moment buffers (``tp_state.rank<r>``, r = position on the model axis) without gathering
    anything, so the resume is exact and needs the same model-axis size; rank 0 adds ``checkpoint.json`` and a gathered
    ``model.safetensors`` for exchange with other runtimes.  With a data axis the groups hold identical state and only
    the first one writes."""
    rank, world = _world(process_info)
    opt = train_state.optimizer
    data_index = rank // tp.world
    if rank == 0:
        checkpoint_dir.mkdir(parents=True, exist_ok=True)
    _barrier(process_info)
    if data_index == 0:
        tensors = {
            "master": opt.flat.master.detach().contiguous().cpu(),
            "exp_avg": opt.exp_avg.detach().contiguous().cpu(),
            "exp_avg_sq": opt.exp_avg_sq.detach().contiguous().cpu(),
            "count": torch.tensor([opt.count], dtype=torch.int64),
        }
        save_file(tensors, str(checkpoint_dir / TP_SHARD_FILE.format(rank=tp.rank)))
    if runtime_state is not None:   # recurrent state holds this rank's heads and this data group's rows
        save_runtime_state(checkpoint_dir / f"runtime_state.rank{rank:05d}.safetensors", runtime_state)
    full = tp.gather_full_parameters(train_state.model)      # collective on every rank of a model-parallel group
    if rank == 0:
        from ..io.names import internal_to_portable

        flat = internal_to_portable({k: v.detach().cpu() for k, v in full.items()}, config)
        save_model_safetensors(checkpoint_dir / MODEL_SAFETENSORS, flat, config,
                               metadata={"checkpoint_step": int(train_state.step), **(metadata or {})})
        payload = {
            "format": "rwkv7m_train_checkpoint", "format_version": 1, "backend": "sharded", "world_size": world,
            "model_parallel": tp.world, "layout": "tensor_parallel", "vocab_parallel": bool(tp.vocab_parallel),
            "step": int(train_state.step), "config": model_config_to_dict(config),
            "rng_key": None if rng_key is None else [int(x) for x in torch.as_tensor(rng_key).reshape(-1).tolist()],
            "dataset_position": dataset_position, "metadata": metadata or {},
        }
    _barrier(process_info)      # every rank's shard is on disk before the file that marks the checkpoint as finished
    if rank == 0:
        write_json_atomic(checkpoint_dir / CHECKPOINT_JSON, payload)
    _barrier(process_info)
    return checkpoint_dir


def _restore_tensor_parallel_shards(checkpoint_dir, train_state, payload, tp):
    if payload.get("layout") != "tensor_parallel":
        raise ValueError("this sharded checkpoint was written by a data-parallel run; restore it without a model axis")
    if int(payload.get("model_parallel", 0)) != tp.world or bool(payload.get("vocab_parallel", False)) != bool(tp.vocab_parallel):
        raise ValueError(
            f"tensor-parallel shards were written for a model axis of {payload.get('model_parallel')} "
            f"(vocab_parallel={payload.get('vocab_parallel')}); restore with the same layout or save with the 'single' backend")
    path = checkpoint_dir / TP_SHARD_FILE.format(rank=tp.rank)
    if not path.exists():
        raise FileNotFoundError(f"sharded checkpoint is missing {path.name}")
    part = load_file(str(path))
    opt = train_state.optimizer
    if part["master"].numel() != opt.flat.master.numel():
        raise ValueError("the flat parameter store of this rank has another size than the saved shard")
    opt.flat.master.copy_(part["master"])
    opt.exp_avg.copy_(part["exp_avg"])
    opt.exp_avg_sq.copy_(part["exp_avg_sq"])
    opt.count = int(part["count"].reshape(-1)[0])
    opt.flat.sync_compute()


def _patch_json(checkpoint_dir, extra: dict):
    path = Path(checkpoint_dir) / CHECKPOINT_JSON
    with open(path, "r", encoding="utf-8") as f:
        payload = json.load(f)
    payload.update(extra)
    write_json_atomic(path, payload)


def restore_distributed_train_state(checkpoint_dir, train_state_template, process_info=None):
    """Restore parameters on every rank and Adam moments into whichever layout the template uses."""
    checkpoint_dir = Path(checkpoint_dir)
    process_info = process_info or {"process_index": 0, "process_count": 1}
    rank, world = _world(process_info)
    config, payload = load_distributed_checkpoint_raw_metadata(checkpoint_dir)
    opt = train_state_template.optimizer
    shard = _moment_shard(train_state_template)
    tp = train_state_template.extras.get("tp")
    if tp is not None and payload.get("backend", "single") == "sharded":
        _restore_tensor_parallel_shards(checkpoint_dir, train_state_template, payload, tp)
        return train_state_template, DistributedCheckpointPayload(
            config, payload, int(payload.get("step", 0)), payload.get("dataset_position"))
    if tp is not None:
        tp.load_full_state(train_state_template, lambda ts: load_train_checkpoint(checkpoint_dir, ts))
        return train_state_template, DistributedCheckpointPayload(
            config, payload, int(payload.get("step", 0)), payload.get("dataset_position"))
    if payload.get("backend", "single") == "sharded" and payload.get("layout") == "tensor_parallel":
        raise ValueError("this checkpoint holds tensor-parallel shards; restore it on a model axis of "
                         f"{payload.get('model_parallel')} or re-save it with the 'single' backend")
    if payload.get("backend", "single") == "sharded":
        # Every rank of the saving run wrote the slice [begin, end) of both moments that it owned.  The restoring run may
        # have another process count or another layout (replicated moments, or other slice bounds): each process reads
        # the files whose ranges overlap what it needs.
        saved_world = int(payload.get("world_size", 1))
        tensors = load_file(str(checkpoint_dir / TRAIN_STATE_FILE))
        from_portable(train_state_template.model,
                      {k[len("model/"):]: v for k, v in tensors.items() if k.startswith("model/")}, strict=True)
        opt.count = int(tensors["optimizer/count"].reshape(-1)[0])
        if shard is not None:
            dst_m, dst_v, need_b, need_e = shard
        else:
            dst_m, dst_v, need_b, need_e = opt.exp_avg, opt.exp_avg_sq, 0, int(opt.exp_avg.numel())
        dst_m.zero_()        # the flat store ends in padding up to a multiple of the process count: zeros on both sides
        dst_v.zero_()
        covered, saved_total = 0, 0
        for r in range(saved_world):
            path = checkpoint_dir / f"optimizer_shard.rank{r:05d}.safetensors"
            if not path.exists():
                raise FileNotFoundError(f"sharded checkpoint is missing {path.name}")
            part = load_file(str(path))
            b, e = (int(x) for x in part["range"].tolist())
            saved_total = max(saved_total, e)
            lo, hi = max(b, need_b), min(e, need_e)
            if lo >= hi:
                continue
            dst_m[lo - need_b:hi - need_b].copy_(part["exp_avg"][lo - b:hi - b])
            dst_v[lo - need_b:hi - need_b].copy_(part["exp_avg_sq"][lo - b:hi - b])
            covered += hi - lo
        expected = max(0, min(need_e, saved_total) - min(need_b, saved_total))
        if covered != expected:
            raise ValueError(f"the optimizer shards cover {covered} of the {expected} saved moment elements this process needs")
        opt.flat.sync_compute()
    else:
        if shard is not None:
            # load the replicated moments into temporary full buffers, then keep only the owned slice
            total = opt.flat.master.numel()
            opt.exp_avg = torch.zeros(total, dtype=torch.float32, device=opt.flat.master.device)
            opt.exp_avg_sq = torch.zeros_like(opt.exp_avg)
        load_train_checkpoint(checkpoint_dir, train_state_template)
        if shard is not None:
            m, v, begin, end = shard
            m.copy_(opt.exp_avg[begin:end])
            v.copy_(opt.exp_avg_sq[begin:end])
            opt.exp_avg = opt.exp_avg_sq = None
    return train_state_template, DistributedCheckpointPayload(
        config, payload, int(payload.get("step", 0)), payload.get("dataset_position")
    )


def restore_distributed_runtime_state(checkpoint_dir, runtime_state_template, process_info=None):
    checkpoint_dir = Path(checkpoint_dir)
    rank = int((process_info or {"process_index": 0})["process_index"])
    per_rank = checkpoint_dir / f"runtime_state.rank{rank:05d}.safetensors"
    if per_rank.exists():
        tmp = checkpoint_dir / RUNTIME_STATE_FILE
        tensors = load_file(str(per_rank))
        from ..state import rwkv_state_from_dict, screen_state_from_dict

        n_layers = len({k.split("/")[0] for k in tensors if k.startswith("layer_")})
        n_scr = len({k.split("/")[0] for k in tensors if k.startswith("screen_")})
        ref = runtime_state_template["rwkv_state"][0].wkv
        return {
            "rwkv_state": tuple(l.to(ref.device) for l in rwkv_state_from_dict(tensors, n_layers)),
            "screen_state": screen_state_from_dict(tensors, n_scr).to(ref.device),
        }
    if (checkpoint_dir / RUNTIME_STATE_FILE).exists():
        return load_train_runtime_state(checkpoint_dir, runtime_state_template)
    return None


def rotate_checkpoints(output_dir, keep_last, process_info, *, protected_paths=None) -> list:
    """Delete all but the newest ``keep_last`` checkpoints (rank 0), never a protected one
    (e.g. the best-eval checkpoint)."""
    if output_dir is None or keep_last is None or keep_last <= 0:
        return []
    if process_info["process_index"] != 0:
        return []
    protected = {Path(p).resolve() for p in (protected_paths or []) if p is not None}
    ckpts = list_checkpoint_dirs(output_dir)
    doomed = [p for p in ckpts[: max(0, len(ckpts) - int(keep_last))] if p.resolve() not in protected]
    for p in doomed:
        shutil.rmtree(p)
    return doomed


# ---- the reference's names for the sharded backend --------------------------------------------------------------------
def _info(process_info):
    if process_info is not None:
        return process_info
    from .mesh import process_info as current

    return current()


def save_orbax_train_state(checkpoint_dir, train_state, *, force=True, process_info=None, config=None):
    """Every process writes its part of the train state (the ``sharded`` backend: the optimizer moments that this rank
    owns; rank 0 adds the model files and ``checkpoint.json``).  Named after the reference's sharded writer
    (src/rwkv7m/distributed/checkpoint.py:146-163); ``force`` is accepted, existing files are always replaced."""
    return _save_checkpoint_dir(checkpoint_dir, train_state, config if config is not None else train_state.config,
                                _info(process_info), backend="sharded")


def load_orbax_train_state(checkpoint_dir, train_state_template, *, process_info=None):
    """Restore what :func:`save_orbax_train_state` wrote into ``train_state_template`` (same process count)."""
    return restore_distributed_train_state(checkpoint_dir, train_state_template, _info(process_info))[0]


def save_orbax_runtime_state(checkpoint_dir, runtime_state, *, force=True, process_info=None):
    """This process's carried recurrent and memory state as ``runtime_state.rank<r>.safetensors``."""
    checkpoint_dir = Path(checkpoint_dir)
    checkpoint_dir.mkdir(parents=True, exist_ok=True)
    rank, _ = _world(_info(process_info))
    path = checkpoint_dir / f"runtime_state.rank{rank:05d}.safetensors"
    save_runtime_state(path, runtime_state)
    return path


def load_orbax_runtime_state(checkpoint_dir, runtime_state_template, *, process_info=None):
    return restore_distributed_runtime_state(checkpoint_dir, runtime_state_template, _info(process_info))
