"""Which kernel owns which collective, and a runtime byte counter.

The reference counts ``all-reduce / all-gather / all-to-all / collective-permute /
reduce-scatter`` in the post-SPMD HLO text (src/rwkv7m/distributed/collectives.py:42-50)
because XLA decides the communication.  Here communication is explicit, so the audit is a
static ownership table plus counters that wrap ``torch.distributed`` while a step runs.
"""

from __future__ import annotations

import contextlib
import re
from collections import Counter

import torch
import torch.distributed as dist

OWNERSHIP = (
    # (parallelism, site, collective, message, where it runs)
    ("dp", "gradient sync (allreduce mode)", "all-reduce", "flat fp32 gradient buffer", "NCCL on the flat buffer"),
    ("dp", "gradient sync (fused mode)", "reduce-scatter", "flat fp32 gradient buffer",
     "dp_reduce_shard_kernel: multimem.ld_reduce / peer loads (csrc/dp_fused.cu)"),
    ("dp", "parameter refresh (fused mode)", "all-gather", "fp32 master + bf16 compute copy",
     "dp_adamw_allgather_kernel epilogue: multimem.st / peer stores (csrc/dp_fused.cu)"),
    ("dp", "global gradient norm (fused mode)", "all-gather of 1 float", "partial sum of squares",
     "dp_barrier_kernel publish (csrc/dp_fused.cu)"),
    ("tp", "time-mix / channel-mix input", "all-gather over time", "[B, T/w, C] -> [B, T, C]", "parallel/tp.py _GatherSeq"),
    ("tp", "att.output / ffn.value result", "reduce-scatter over time", "[B, T, C] -> [B, T/w, C]",
     "parallel/tp.py _ReduceScatterSeq"),
    ("tp", "replicated-parameter gradients", "all-reduce", "LayerNorm, token-shift mixes, LoRA-down, embedding",
     "TensorParallel.reduce_replicated_grads"),
    ("tp", "vocab-parallel loss", "all-reduce x3", "max, sum-exp, target logit per token", "vocab_parallel_cross_entropy"),
    ("tp", "global gradient norm", "all-reduce", "1 float", "TensorParallel.grad_norm_sq_reduce"),
    ("any", "metrics", "all-reduce", "loss scalars", "DataParallelTrainer.train_step"),
)

_HLO_KINDS = ("all-reduce", "all-gather", "all-to-all", "collective-permute", "reduce-scatter")


class CollectiveAudit(dict):
    """Counts per collective kind; a mapping (``audit["all-reduce"]``) with the reference's record interface on top
    (``counts``, ``total``, ``to_dict()``; src/rwkv7m/distributed/collectives.py:19-29)."""

    @property
    def counts(self) -> dict:
        return dict(self)

    @property
    def total(self) -> int:
        return sum(self.values())

    def to_dict(self) -> dict:
        return {"counts": dict(self), "total": self.total}


def audit_collectives(text: str) -> CollectiveAudit:
    """Count collective op names in a textual program dump (kept for parity with HLO-based audits)."""
    return CollectiveAudit({kind: len(re.findall(rf"\b{re.escape(kind)}(?:-start)?\b", text)) for kind in _HLO_KINDS})


def compiler_ir_text(program, *, dialect: str = "hlo") -> str:
    """Text of a program to audit.  Accepts a string, an object with ``as_text()`` / ``compiler_ir()`` (a lowered or
    compiled computation of a tracing compiler), or the record of :func:`count_collectives`, whose calls are written one
    per line under their HLO names so that the same text audit reads both."""
    if isinstance(program, str):
        return program
    if isinstance(program, dict) and "calls" in program:
        names = {"all_reduce": "all-reduce", "all_gather": "all-gather", "all_gather_into_tensor": "all-gather",
                 "reduce_scatter_tensor": "reduce-scatter", "all_to_all_single": "all-to-all", "broadcast": "broadcast"}
        lines = []
        for call, n in sorted(program["calls"].items()):
            lines += [f"%c = {names.get(call, call)}(%x)"] * int(n)
        return "\n".join(lines)
    if hasattr(program, "compiler_ir"):
        ir = program.compiler_ir(dialect=dialect)
        as_hlo_text = getattr(ir, "as_hlo_text", None)
        return as_hlo_text() if as_hlo_text is not None else str(ir)
    as_text = getattr(program, "as_text", None)
    if as_text is None:
        raise TypeError("object exposes neither compiler_ir() nor as_text()")
    return as_text()


def audit_lowered_collectives(program, *, dialect: str = "hlo") -> CollectiveAudit:
    return audit_collectives(compiler_ir_text(program, dialect=dialect))


def ownership_table(parallelism: str | None = None) -> list:
    rows = [dict(zip(("parallelism", "site", "collective", "message", "owner"), r)) for r in OWNERSHIP]
    return [r for r in rows if parallelism in (None, r["parallelism"], "any") or r["parallelism"] == "any"]


@contextlib.contextmanager
def count_collectives():
    """Counts calls and payload bytes of the torch.distributed collectives issued inside the block."""
    counts, nbytes = Counter(), Counter()
    names = ("all_reduce", "all_gather", "all_gather_into_tensor", "reduce_scatter_tensor", "broadcast", "all_to_all_single")
    originals = {n: getattr(dist, n) for n in names if hasattr(dist, n)}

    def wrap(name, fn):
        def inner(*args, **kwargs):
            counts[name] += 1
            for a in args[:2]:
                if isinstance(a, torch.Tensor):
                    nbytes[name] += a.numel() * a.element_size()
                    break
            return fn(*args, **kwargs)
        return inner

    for n, fn in originals.items():
        setattr(dist, n, wrap(n, fn))
    try:
        yield {"calls": counts, "bytes": nbytes}
    finally:
        for n, fn in originals.items():
            setattr(dist, n, fn)
