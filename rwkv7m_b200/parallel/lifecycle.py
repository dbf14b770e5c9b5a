"""Create -> step -> save -> restore-in-a-new-process -> step probe.

Counterpart of the reference's NNX lifecycle probe (src/rwkv7m/distributed/nnx_lifecycle.py:10-144):
a deliberately tiny model goes through the full life of a training state so the checkpoint path can be
verified across processes without a real run.  ``create`` writes a checkpoint and the value it expects
the next step to produce; ``restore`` (run in a different process) must reproduce that value.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

from ..config import tiny_config
from ..io.checkpoint import load_train_checkpoint, save_train_checkpoint
from ..train.train_step import generate_toy_batch, initialize_train_state, train_step
from ..state import init_rwkv_state, init_screen_state

PROBE_FILE = "lifecycle_probe.json"


def _probe_config():
    cfg = tiny_config(vocab_size=64, d_model=32, n_layers=2, n_heads=2, head_size=16)
    cfg.warmup_steps = 0
    return cfg


def _one_step(ts, cfg, seed):
    batch = generate_toy_batch(seed, 2, 6, cfg.vocab_size)
    rs = init_rwkv_state(2, cfg)
    ss = init_screen_state(2, cfg.screening)
    ts, _, _, metrics = train_step(ts, batch, rs, ss)
    return ts, float(metrics["loss"])


def create_lifecycle_checkpoint(directory, seed: int = 0) -> dict:
    directory = Path(directory)
    cfg = _probe_config()
    ts = initialize_train_state(seed, cfg, total_steps=10)
    ts, loss0 = _one_step(ts, cfg, 1)
    save_train_checkpoint(directory / "ckpt-00000001", ts, cfg, rng_key=[0, seed], dataset_position={"step": 1})
    ts, loss1 = _one_step(ts, cfg, 2)  # what a faithful restore must reproduce
    checksum = float(sum(p.detach().double().sum() for p in ts.model.parameters()))
    probe = {"seed": seed, "loss_after_create": loss0, "expected_next_loss": loss1, "expected_checksum": checksum,
             "param_count": sum(p.numel() for p in ts.model.parameters())}
    (directory / PROBE_FILE).write_text(json.dumps(probe, indent=2))
    return probe


def restore_lifecycle_checkpoint(directory, rtol: float = 1e-5) -> dict:
    directory = Path(directory)
    probe = json.loads((directory / PROBE_FILE).read_text())
    cfg = _probe_config()
    ts = initialize_train_state(probe["seed"] + 1000, cfg, total_steps=10)  # different init: restore must overwrite it
    ts, _, payload = load_train_checkpoint(directory / "ckpt-00000001", ts)
    assert int(payload["step"]) == 1 and ts.step == 1
    ts, loss1 = _one_step(ts, cfg, 2)
    checksum = float(sum(p.detach().double().sum() for p in ts.model.parameters()))
    ok = (abs(loss1 - probe["expected_next_loss"]) <= rtol * max(1.0, abs(loss1))
          and abs(checksum - probe["expected_checksum"]) <= rtol * max(1.0, abs(checksum)))
    return {"ok": bool(ok), "next_loss": loss1, "expected_next_loss": probe["expected_next_loss"],
            "checksum": checksum, "expected_checksum": probe["expected_checksum"], "restored_step": int(payload["step"])}


# ---------------------------------------------------------------------------------------------------------------------
# Sharded probe: a two-projection tensor-parallel module goes through initialise -> step -> sharded save -> restore ->
# step, with the model axis spanning every process (reference: src/rwkv7m/distributed/nnx_lifecycle.py:10-144 and
# src/rwkv7m/cli/verify_nnx_lifecycle.py:38-93).  Each process holds its column / row slices only, writes its own
# shard file, and a restore may use a different number of processes: the slices are cut again from the shard files.
# ---------------------------------------------------------------------------------------------------------------------
SHARD_META = "sharding_probe.json"

# leaf name -> (sharded dimension or None, logical axes as the report prints them)
_PROBE_LAYOUT = {
    "in_proj.weight": (0, ("model", None)),     # column-parallel: output features split, stored [out, in]
    "in_proj.bias": (0, ("model",)),
    "out_proj.weight": (1, (None, "model")),    # row-parallel: input features split
    "out_proj.bias": (None, (None,)),
}


def _group_info(group=None):
    import torch.distributed as dist

    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


class ShardingProbe(torch.nn.Module):
    """``out_proj(relu(in_proj(x)))`` with ``in_proj`` split by output feature and ``out_proj`` by input feature; one
    all-reduce of the partial outputs per forward.  Initial values are drawn for the full matrices from the seed and then
    sliced, so every process count starts from the same model."""

    def __init__(self, width: int, *, seed: int = 0, group=None, device="cpu"):
        super().__init__()
        rank, world = _group_info(group)
        if width <= 0 or width % world != 0:
            raise ValueError("width must be positive and divisible by the model axis size")
        self.width, self.group, self.rank, self.world = width, group, rank, world
        g = torch.Generator().manual_seed(seed)
        w_in = torch.randn(width, width, generator=g) / width ** 0.5
        w_out = torch.randn(width, width, generator=g) / width ** 0.5
        s = width // world
        lo, hi = rank * s, (rank + 1) * s
        self.in_proj = torch.nn.Linear(width, s, device=device)
        self.out_proj = torch.nn.Linear(s, width, device=device)
        with torch.no_grad():
            self.in_proj.weight.copy_(w_in[lo:hi])
            self.in_proj.bias.zero_()
            self.out_proj.weight.copy_(w_out[:, lo:hi])
            self.out_proj.bias.zero_()

    def forward(self, x):
        h = torch.relu(self.in_proj(x))
        partial = torch.nn.functional.linear(h, self.out_proj.weight)
        if self.world > 1:
            partial = _AllReduceSum.apply(partial, self.group)
        return partial + self.out_proj.bias


class _AllReduceSum(torch.autograd.Function):
    """Sum over the model axis in forward; the cotangent is already the same on every process, so backward passes it on."""

    @staticmethod
    def forward(ctx, x, group):
        import torch.distributed as dist

        y = x.clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, dy):
        return dy, None


def initialize_sharding_probe(*, width: int = 8, learning_rate: float = 1e-3, seed: int = 0, group=None, device="cpu"):
    model = ShardingProbe(width, seed=seed, group=group, device=device)
    optimizer = torch.optim.Adam(model.parameters(), lr=learning_rate)
    return model, optimizer


def train_sharding_probe_step(model, optimizer, inputs, targets):
    """One mean-squared-error step; every slice stays where it is."""
    optimizer.zero_grad(set_to_none=True)
    loss = torch.mean(torch.square(model(inputs) - targets))
    loss.backward()
    optimizer.step()
    return float(loss.detach())


def probe_optimizer_step(optimizer) -> int:
    steps = [int(s["step"]) for s in optimizer.state.values() if "step" in s]
    return max(steps) if steps else 0


def sharding_summary(model, optimizer) -> dict:
    """Per leaf (parameters and both Adam moments): global shape, this process's shape, dtype, the split and the logical axes."""
    out = {}
    named = dict(model.named_parameters())
    for name, p in named.items():
        dim, axes = _PROBE_LAYOUT[name]
        shape = list(p.shape)
        if dim is not None:
            shape[dim] *= model.world
        row = {"shape": shape, "local_shape": list(p.shape), "dtype": str(p.dtype).replace("torch.", ""),
               "sharding": str(tuple(axes)), "logical_axes": list(axes)}
        out[f"model/{name}"] = row
        state = optimizer.state.get(p, {})
        for moment in ("exp_avg", "exp_avg_sq"):
            if moment in state:
                out[f"optimizer/{moment}/{name}"] = dict(row, dtype=str(state[moment].dtype).replace("torch.", ""))
    return out


def save_sharding_probe_checkpoint(checkpoint_dir, model, optimizer, extra: dict | None = None):
    """Every process writes ``shard-<rank>-of-<world>.safetensors`` (its slices of the parameters and of both moments);
    process 0 also writes the layout record."""
    from safetensors.torch import save_file

    checkpoint_dir = Path(checkpoint_dir).resolve()
    checkpoint_dir.mkdir(parents=True, exist_ok=True)
    tensors = {}
    for name, p in model.named_parameters():
        tensors[f"model/{name}"] = p.detach().cpu().contiguous()
        state = optimizer.state.get(p, {})
        for moment in ("exp_avg", "exp_avg_sq"):
            if moment in state:
                tensors[f"optimizer/{moment}/{name}"] = state[moment].detach().cpu().contiguous()
    save_file(tensors, str(checkpoint_dir / f"shard-{model.rank:05d}-of-{model.world:05d}.safetensors"))
    if model.rank == 0:
        meta = {"width": model.width, "world": model.world, "optimizer_step": probe_optimizer_step(optimizer),
                "layout": {k: {"dim": v[0], "axes": list(v[1])} for k, v in _PROBE_LAYOUT.items()}}
        meta.update(extra or {})
        (checkpoint_dir / SHARD_META).write_text(json.dumps(meta, indent=2))
    if model.world > 1:
        import torch.distributed as dist

        dist.barrier(group=model.group)
    return checkpoint_dir


def _assemble(checkpoint_dir: Path, saved_world: int) -> dict:
    from safetensors.torch import load_file

    shards = [load_file(str(checkpoint_dir / f"shard-{r:05d}-of-{saved_world:05d}.safetensors")) for r in range(saved_world)]
    full = {}
    for key in shards[0]:
        dim = _PROBE_LAYOUT[key.split("/")[-1]][0]
        full[key] = shards[0][key] if dim is None else torch.cat([s[key] for s in shards], dim=dim)
    return full


def restore_sharding_probe_checkpoint(checkpoint_dir, *, width: int | None = None, learning_rate: float = 1e-3,
                                      seed: int = 0, group=None, device="cpu"):
    """Rebuild model and optimizer from the shard files.  With the process count of the save each process reads only its
    own file; with another count the full tensors are put together from all files and cut again."""
    from safetensors.torch import load_file

    checkpoint_dir = Path(checkpoint_dir).resolve()
    meta = json.loads((checkpoint_dir / SHARD_META).read_text())
    if width is not None and width != meta["width"]:
        raise ValueError(f"checkpoint holds a probe of width {meta['width']}, not {width}")
    model, optimizer = initialize_sharding_probe(width=meta["width"], learning_rate=learning_rate, seed=seed + 1000,
                                                 group=group, device=device)   # another start: the restore must replace it
    saved_world = int(meta["world"])
    if saved_world == model.world:
        mine = load_file(str(checkpoint_dir / f"shard-{model.rank:05d}-of-{saved_world:05d}.safetensors"))
    else:
        mine = {}
        for key, value in _assemble(checkpoint_dir, saved_world).items():
            dim = _PROBE_LAYOUT[key.split("/")[-1]][0]
            mine[key] = value if dim is None else value.chunk(model.world, dim=dim)[model.rank].contiguous()
    step = torch.tensor(float(meta["optimizer_step"]))
    with torch.no_grad():
        for name, p in model.named_parameters():
            p.copy_(mine[f"model/{name}"])
            optimizer.state[p] = {"step": step.clone(), "exp_avg": mine[f"optimizer/exp_avg/{name}"].to(p.device).clone(),
                                  "exp_avg_sq": mine[f"optimizer/exp_avg_sq/{name}"].to(p.device).clone()}
    return model, optimizer, meta


def run_sharding_probe(checkpoint_dir, mode: str, *, width: int | None = None, learning_rate: float = 1e-3, seed: int = 0,
                       group=None, device="cpu") -> dict:
    """The whole probe of one process.  ``create``: initialise, one step, save, then one more step whose loss is recorded as
    what a faithful restore has to reproduce.  ``restore``: load, one step, compare with that record."""
    from .environment import runtime_version_manifest

    rank, world = _group_info(group)
    checkpoint_dir = Path(checkpoint_dir).resolve()
    if mode == "create":
        width = width if width is not None else max(8, world)
        model, optimizer = initialize_sharding_probe(width=width, learning_rate=learning_rate, seed=seed, group=group,
                                                     device=device)
        meta = None
    elif mode == "restore":
        model, optimizer, meta = restore_sharding_probe_checkpoint(checkpoint_dir, width=width, learning_rate=learning_rate,
                                                                   seed=seed, group=group, device=device)
        width = model.width
    else:
        raise ValueError("mode must be 'create' or 'restore'")
    before = sharding_summary(model, optimizer)
    inputs = torch.arange(2 * width, dtype=torch.float32, device=device).reshape(2, width)
    targets = torch.zeros_like(inputs)
    loss = train_sharding_probe_step(model, optimizer, inputs, targets)
    after = sharding_summary(model, optimizer)
    report = {"mode": mode, "loss": loss, "optimizer_step": probe_optimizer_step(optimizer),
              "mesh": {"axis_names": ["data", "model"], "shape": {"data": 1, "model": world}},
              "sharding_before": before, "sharding_after": after, "environment": runtime_version_manifest(),
              "checkpoint_dir": str(checkpoint_dir), "process_index": rank}
    if mode == "create":
        import copy

        saved_opt_state = copy.deepcopy(optimizer.state_dict())
        saved_params = [p.detach().clone() for p in model.parameters()]
        expected = train_sharding_probe_step(model, optimizer, inputs, targets)   # what the restored state must produce
        with torch.no_grad():
            for p, v in zip(model.parameters(), saved_params):
                p.copy_(v)
        optimizer.load_state_dict(saved_opt_state)
        save_sharding_probe_checkpoint(checkpoint_dir, model, optimizer, {"expected_next_loss": expected, "seed": seed})
        report["expected_next_loss"] = expected
        report["ok"] = True
    else:
        want = float(meta["expected_next_loss"])
        report["expected_next_loss"] = want
        report["ok"] = bool(abs(loss - want) <= 1e-5 * max(1.0, abs(want)))
    return report
