"""Command-line tools run in-process on tiny models (CPU)."""

import csv
import json
import os
from pathlib import Path

import numpy as np
import pytest
import torch

from rwkv7m_b200.cli import eval_binidx, generate, make_binidx, plan_scale, train_binidx, train_binidx_distributed
from rwkv7m_b200.cli.common import default_bank_ids, parse_args_with_config

TINY = ["--vocab-size", "300", "--d-model", "32", "--d-ffn", "64", "--n-layers", "2", "--n-heads", "2",
        "--head-size", "16", "--d-slot", "16", "--d-k", "8", "--d-v", "8", "--device", "cpu"]


def test_config_file_supplies_defaults_and_rejects_unknown_keys(tmp_path):
    import argparse

    p = argparse.ArgumentParser()
    p.add_argument("--alpha", type=int, required=True)
    p.add_argument("--beta", type=int, default=1)
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps({"alpha": 5}))
    args = parse_args_with_config(p, ["--config", str(cfg), "--beta", "3"])
    assert (args.alpha, args.beta) == (5, 3)
    cfg.write_text(json.dumps({"gamma": 1}))
    p2 = argparse.ArgumentParser()
    p2.add_argument("--alpha", type=int, default=0)
    with pytest.raises(ValueError):
        parse_args_with_config(p2, ["--config", str(cfg)])


def test_default_bank_ids():
    assert default_bank_ids(1) == (0,)
    assert default_bank_ids(2) == (0, 2)
    assert default_bank_ids(4) == (0, 0, 1, 2)
    assert default_bank_ids(16) == (0,) * 8 + (1,) * 4 + (2,) * 4


def test_train_save_resume_and_eval(tiny_binidx, tmp_path):
    out = tmp_path / "run"
    base = ["--data-file", tiny_binidx, "--ctx-len", "4", "--batch-size", "2", "--print-every", "0",
            "--output-dir", str(out)] + TINY
    args = train_binidx.parse_args(base + ["--steps", "1"])
    ts, rt, ckpt = train_binidx.run_training(args)
    assert ckpt.name == "ckpt-00000001" and (ckpt / "model.safetensors").exists()
    assert json.loads((ckpt / "checkpoint.json").read_text())["step"] == 1
    args = train_binidx.parse_args(base + ["--steps", "1", "--resume", str(ckpt)])
    ts2, _, ckpt2 = train_binidx.run_training(args)
    assert int(ts2.step) == 2 and ckpt2.name == "ckpt-00000002"
    m = eval_binidx.evaluate_binidx(eval_binidx.parse_args(
        ["--data-file", tiny_binidx, "--checkpoint", str(ckpt2), "--ctx-len", "4", "--steps", "2",
         "--print-every", "0", "--device", "cpu"]))
    assert m["loss"] > 0 and m["perplexity"] == pytest.approx(np.exp(min(m["loss"], 20.0)))


def test_carry_state_requires_sequential_and_writes_runtime_state(tiny_binidx, tmp_path):
    base = ["--data-file", tiny_binidx, "--ctx-len", "4", "--batch-size", "2", "--steps", "2", "--print-every", "0",
            "--output-dir", str(tmp_path / "r")] + TINY
    with pytest.raises(ValueError):
        train_binidx.run_training(train_binidx.parse_args(base + ["--carry-state"]))
    _, rt, ckpt = train_binidx.run_training(
        train_binidx.parse_args(base + ["--carry-state", "--sampling-mode", "sequential"]))
    assert (ckpt / "runtime_state.safetensors").exists()
    assert float(rt.rwkv_state[0].wkv.abs().sum()) > 0


def test_make_binidx_and_generate(tmp_path, tiny_binidx):
    src = tmp_path / "toy.jsonl"
    src.write_text("\n".join(json.dumps({"text": t}) for t in ["hello world", "RWKV は速い", "abc"]) + "\n")
    stats = make_binidx.build_binidx(str(src), str(tmp_path / "toy"), epochs=2, seed=1)
    assert stats["items"] == 6 and stats["tokens"] > 6
    out = tmp_path / "g"
    args = train_binidx.parse_args(["--data-file", tiny_binidx, "--ctx-len", "4", "--steps", "1", "--print-every", "0",
                                    "--output-dir", str(out), "--vocab-size", "65536", "--d-model", "32", "--d-ffn",
                                    "64", "--n-layers", "1", "--n-heads", "2", "--head-size", "16", "--no-screening",
                                    "--device", "cpu"])
    _, _, ckpt = train_binidx.run_training(args)
    text = generate.main(["--checkpoint", str(ckpt), "--prompt", "hi", "--max-new-tokens", "3", "--temperature", "0",
                          "--device", "cpu"])
    assert text.startswith("hi")
    # several prompts (flags and a file), several samples each, a JSON record of everything
    (tmp_path / "prompts.txt").write_text("abc\n\nRWKV\n", encoding="utf-8")
    texts = generate.main(["--checkpoint", str(ckpt), "--prompt", "hi", "--prompt", "yo", "--prompt-file",
                           str(tmp_path / "prompts.txt"), "--num-samples", "2", "--max-new-tokens", "2", "--temperature", "0.7",
                           "--continuation-only", "--json-out", str(tmp_path / "gen" / "out.json"), "--device", "cpu"])
    record = json.loads((tmp_path / "gen" / "out.json").read_text(encoding="utf-8"))
    assert len(texts) == 8 and [s["prompt"] for s in record["samples"]] == ["hi", "hi", "yo", "yo", "abc", "abc", "RWKV", "RWKV"]
    assert [s["seed"] for s in record["samples"][:2]] == [42, 43] and record["settings"]["temperature"] == 0.7
    with pytest.raises(SystemExit):
        generate.parse_args(["--checkpoint", str(ckpt)])
    # the same checkpoint served by two tensor-parallel processes gives the same greedy continuation
    import socket
    import subprocess
    import sys

    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    root = Path(__file__).resolve().parents[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "rwkv7m_b200.cli.generate", "--checkpoint", str(ckpt), "--prompt", "hi",
           "--max-new-tokens", "3", "--temperature", "0", "--device", "cpu", "--model-axis-size", "2",
           "--json-out", str(tmp_path / "tp.json")]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(root),
                         env=dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-2000:]
    assert json.loads((tmp_path / "tp.json").read_text(encoding="utf-8"))["samples"][0]["text"] == text
    # and with the prefill of a longer prompt split along time over two processes that each hold the whole model
    prompt = "hello world, hello world"
    want = generate.main(["--checkpoint", str(ckpt), "--prompt", prompt, "--max-new-tokens", "3", "--temperature", "0",
                          "--device", "cpu"])
    cmd = cmd[:cmd.index("--checkpoint")] + ["--checkpoint", str(ckpt), "--prompt", prompt, "--max-new-tokens", "3",
                                             "--temperature", "0", "--device", "cpu", "--context-parallel-size", "2",
                                             "--json-out", str(tmp_path / "cp.json")]
    cmd[cmd.index("--master-port") + 1] = str(port + 1 if port < 65000 else port - 1)
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(root),
                         env=dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-2000:]
    assert json.loads((tmp_path / "cp.json").read_text(encoding="utf-8"))["samples"][0]["text"] == want


def test_plan_scale_outputs_exact_counts(capsys):
    est = plan_scale.main(["--model-preset", "0.185b", "--model-axis-size", "1", "--optimizer-shards", "8"])
    assert est.parameter_summary.total == 184_985_222
    assert est.optimizer_state_bytes == -(-184_985_222 * 2 * 4 // 8)
    report = json.loads(capsys.readouterr().out)
    assert "limitations" in report["estimate"] and "torch" in json.dumps(report["environment"])
    memory = plan_scale.build_report(plan_scale.parse_args(["--model-preset", "0.185b", "--model-axis-size", "2",
                                                            "--dtype-profile", "stability"]))
    assert memory["estimate"]["dtype_policy"] != report["estimate"]["dtype_policy"]


def test_distributed_trainer_single_process_artifacts(tiny_binidx, tmp_path):
    out = tmp_path / "dp"
    argv = ["--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2", "--steps", "4",
            "--print-every", "0", "--output-dir", str(out), "--save-every", "1", "--keep-last-checkpoints", "2",
            "--eval-every", "2", "--save-best-checkpoint", "--summary-every", "1", "--disable-python-gc"] + TINY
    ts, rt, summary = train_binidx_distributed.run_distributed_training(train_binidx_distributed.parse_args(argv))
    assert summary["status"] == "completed" and summary["completed_steps"] == 4
    assert json.loads((out / "run_summary.json").read_text())["status"] == "completed"
    assert (out / "run_config.json").exists() and (out / "best_eval.json").exists()
    lines = [json.loads(l) for l in (out / "metrics.jsonl").read_text().splitlines()]
    assert sum(l["split"] == "train" for l in lines) == 4 and sum(l["split"] == "eval" for l in lines) == 2
    kept = sorted(p.name for p in out.iterdir() if p.name.startswith("ckpt-"))
    best = Path(json.loads((out / "best_eval.json").read_text())["checkpoint"]).name
    assert "ckpt-00000004" in kept and best in kept and len(kept) <= 3
    # resume: two more updates
    ts2, _, s2 = train_binidx_distributed.run_distributed_training(train_binidx_distributed.parse_args(
        argv[:6] + ["--steps", "2"] + argv[8:] + ["--resume", str(out / "ckpt-00000004")]))
    assert int(ts2.step) == 6 and s2["start_step"] == 4


def test_compare_variants_plan_run_summarize(tiny_binidx, tmp_path):
    from rwkv7m_b200.cli import compare_variants

    model = ["--d-model", "32", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64",
             "--vocab-size", "300", "--n-slots", "4", "--d-slot", "16", "--d-k", "8", "--d-v", "8", "--screened-layers", "1"]
    plan = compare_variants.plan_variants(model)
    v = plan["variants"]
    C, dk, dv, ds, M = 32, 8, 8, 16, 4
    read_extra = 2 * C + C * dk + ds * dk + ds * dv + dv * C + C * C + C + (2 * C + ds) * ds + ds + 2 + M * ds + 3
    assert v["local_read_screening"]["trainable_params"] - v["local_core_baseline"]["trainable_params"] == read_extra
    assert v["local_mechanism"]["trainable_params"] - v["local_read_screening"]["trainable_params"] == 2 * C * dk + ds * dk + 1
    assert v["local_param_control"]["trainable_params"] >= plan["param_target"] > v["local_core_baseline"]["trainable_params"]
    assert v["local_param_control"]["d_ffn"] % 32 == 0 and v["local_param_control"]["use_screening"] == 0

    root = tmp_path / "cmp"
    train = ["--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2", "--steps", "4", "--print-every", "0",
             "--eval-every", "2", "--summary-every", "0"]
    out = compare_variants.run_variants(root, model + train)
    assert all(s["status"] == "completed" for s in out["summaries"].values()) and len(out["summaries"]) == 4
    summary = compare_variants.summarize(root, tokens_per_step=8, loss_targets=[100.0])
    assert set(summary) == set(compare_variants.VARIANT_ORDER)
    for row in summary.values():
        assert row["train_steps"] == 4 and row["final_eval_loss"] is not None and row["eval_loss_auc_mean"] is not None
        assert row["targets"]["100"]["step"] == 2 and "local_core_baseline_final" in row["targets"]
    assert (root / "summary.csv").exists() and (root / "parameter_counts.csv").exists()


def test_compare_variants_corpus_and_upstream_arm(tmp_path):
    """``corpus`` tokenises a local text file into train / validation binidx; ``--with-upstream`` adds the
    upstream-protocol arm next to the local variants and the summary lists it."""
    from rwkv7m_b200.cli import compare_variants

    corpus = tmp_path / "corpus.txt"
    corpus.write_text("\n".join(f"document {i}: the quick brown fox jumps over the lazy dog {i} times." for i in range(40)))
    root = tmp_path / "cmp2"
    stats = compare_variants.prepare_corpus(corpus, root, ctx_len=8, validation_fraction=0.1, epochs=2)
    assert stats["validation"]["documents"] == 4 and stats["train"]["documents"] == 36
    assert stats["train"]["items"] == 72 and stats["train"]["magic_prime"] % 3 == 2
    model = ["--d-model", "32", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64",
             "--vocab-size", "65536", "--n-slots", "4", "--d-slot", "16", "--d-k", "8", "--d-v", "8", "--screened-layers", "1"]
    train = ["--data-file", stats["train"]["prefix"], "--ctx-len", "8",
             "--global-batch-size", "2", "--steps", "3", "--print-every", "0", "--eval-every", "3", "--summary-every", "0",
             "--device", "cpu"]
    out = compare_variants.run_variants(root, model + train, variants=("local_core_baseline",), with_upstream=True)
    assert out["summaries"][compare_variants.UPSTREAM_VARIANT]["status"] == "completed"
    summary = compare_variants.summarize(root, tokens_per_step=16)
    assert set(summary) == {"local_core_baseline", compare_variants.UPSTREAM_VARIANT}
    assert summary[compare_variants.UPSTREAM_VARIANT]["train_steps"] == 3


def test_distributed_trainer_accepts_a_model_axis(tiny_binidx, tmp_path):
    """``--mesh-axis-names data model --mesh-axis-sizes 1 2``: two gloo ranks train tensor-parallel through the
    trainer CLI, write an un-sharded checkpoint, and a single process resumes from it."""
    import os
    import socket
    import subprocess
    import sys

    root = Path(__file__).resolve().parents[1]
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = tmp_path / "tp_run"
    tiny = ["--d-model", "32", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64",
            "--vocab-size", "300", "--no-screening"]
    common = ["--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2", "--print-every", "0",
              "--output-dir", str(out), "--save-every", "2", "--device", "cpu"] + tiny
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "rwkv7m_b200.cli.train_binidx_distributed", "--steps", "2",
           "--mesh-axis-names", "data", "model", "--mesh-axis-sizes", "1", "2", "--collective-timeout-s", "60"] + common
    env = dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES="")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=str(root))
    assert res.returncode == 0, res.stderr[-2000:]
    summary = json.loads((out / "run_summary.json").read_text())
    assert summary["status"] == "completed" and summary["mesh"] == {"data": 1, "model": 2}
    cfg = json.loads((out / "run_config.json").read_text())
    assert cfg["partition"]["world"] == 2
    # the same two steps in one process give the same loss curve (tensor parallelism changes the layout, not the math)
    single = tmp_path / "single_run"
    argv = ["--steps", "2"] + [a if a != str(out) else str(single) for a in common]
    train_binidx_distributed.run_distributed_training(train_binidx_distributed.parse_args(argv))
    a = [json.loads(l) for l in (out / "metrics.jsonl").read_text().splitlines() if '"train"' in l]
    b = [json.loads(l) for l in (single / "metrics.jsonl").read_text().splitlines() if '"train"' in l]
    assert [r["loss"] for r in a] == pytest.approx([r["loss"] for r in b], rel=1e-4)
    # and the checkpoint is un-sharded: a single process resumes from it
    ts, _, s2 = train_binidx_distributed.run_distributed_training(
        train_binidx_distributed.parse_args(["--steps", "1", "--resume", str(out / "ckpt-00000002")] + common))
    assert s2["status"] == "completed" and int(ts.step) == 3


def test_upstream_single_device_trainer_protocol(tiny_binidx, tmp_path):
    """The upstream-protocol loop: learning-rate rule, optimizer groups, sampler, artefacts, weights that move."""
    from rwkv7m_b200.cli import train_upstream_single_gpu as up
    from rwkv7m_b200.data.dataset import create_binidx_dataset

    assert up.upstream_learning_rate(0, lr_init=1e-3, lr_final=1e-5, warmup_steps=10, total_steps=100) == pytest.approx(1e-5)
    assert up.upstream_learning_rate(10, lr_init=1e-3, lr_final=1e-5, warmup_steps=10, total_steps=100) == pytest.approx(1e-3)
    assert up.upstream_learning_rate(100, lr_init=1e-3, lr_final=1e-5, warmup_steps=10, total_steps=100) == pytest.approx(1e-5)
    assert up.optimizer_group("blocks.0.att.w0", 1, 0.001) == "2x"
    assert up.optimizer_group("blocks.0.att.key.weight", 2, 0.001) == "decay"
    assert up.optimizer_group("blocks.0.att.key.weight", 2, 0.0) == "1x"
    assert up.optimizer_group("blocks.0.att.w1", 2, 0.001) == "1x"
    ds = create_binidx_dataset(tiny_binidx, ctx_len=4)
    prime = ds.magic_prime
    # the trainer's sampler walks the same cubic permutation as the framework's dataset
    assert [up.sample_offset(i, magic_prime=prime, ctx_len=4) for i in range(5)] == [ds.sample_offset(i) for i in range(5)]
    ds.close()
    out = tmp_path / "up"
    last = up.main(["--data-file", tiny_binidx, "--output-dir", str(out), "--steps", "12", "--global-batch-size", "4",
                    "--micro-batch-size", "2", "--ctx-len", "4", "--magic-prime", str(prime), "--n-layer", "2",
                    "--n-embd", "32", "--dim-ffn", "64", "--vocab-size", "300", "--head-size", "16", "--precision", "fp32",
                    "--warmup-steps", "2", "--lr-init", "3e-3", "--device", "cpu", "--save-every", "6"])
    rows = [json.loads(l) for l in (out / "metrics.jsonl").read_text().splitlines()]
    assert len(rows) == 12 and rows[-1]["step"] == 12
    assert all(r["loss"] == r["loss"] and r["loss"] < 7.0 and r["grad_norm"] > 0 for r in rows)   # near ln(300) = 5.7
    assert rows[0]["lr"] == pytest.approx(3e-3 * 0.01) and rows[2]["lr"] == pytest.approx(3e-3)
    w0, w1 = torch.load(out / "rwkv-init.pth"), torch.load(out / "rwkv-final.pth")
    assert set(w0) == set(w1) and float((w0["blocks.0.att.key.weight"] - w1["blocks.0.att.key.weight"]).abs().max()) > 0
    cfg = json.loads((out / "run_config.json").read_text())
    assert cfg["gradient_accumulation_steps"] == 2 and "blocks.0.att.w0" in cfg["optimizer_groups"]["2x"]
    assert (out / "rwkv-6.pth").exists() and (out / "rwkv-final.pth").exists()
    assert json.loads((out / "run_summary.json").read_text())["status"] == "completed"
    assert last["tokens"] == 12 * 4 * 4


def test_preset_execution_controls_are_opt_in_overrides():
    """A preset brings its own recompute / chunking choices; the trainer's flags override each one in both directions
    (scenario of the reference's tests/test_unified_model_scale.py:195-242)."""
    from rwkv7m_b200.cli.common import build_config

    base = ["--data-file", "unused", "--model-preset", "0.185b", "--ctx-len", "512", "--global-batch-size", "1", "--steps", "0"]
    parse = train_binidx_distributed.parse_args
    preset = build_config(parse(base))
    assert (preset.remat_blocks, preset.sequence_chunk_size, preset.head_chunk_size) == (True, 128, None)
    plain = build_config(parse(base + ["--no-remat-blocks", "--no-sequence-chunking", "--no-head-chunking"]))
    assert (plain.remat_blocks, plain.sequence_chunk_size, plain.head_chunk_size) == (False, None, 512)
    chosen = build_config(parse(base + ["--remat-blocks", "--sequence-chunk-size", "256", "--head-chunk-size", "512"]))
    assert (chosen.remat_blocks, chosen.sequence_chunk_size, chosen.head_chunk_size) == (True, 256, 512)


def test_model_axis_run_with_the_sharded_backend_resumes_exactly(tiny_binidx, tmp_path):
    """The reference's documented model-parallel command uses ``--checkpoint-backend orbax``
    (README "Model-size presets and the NNX scale path"): two ranks on a model axis write one shard file each (flat master
    and both moments of that rank, nothing gathered) plus a gathered ``model.safetensors``; a resume on the same axis
    continues with the loss curve of an uninterrupted run, carried runtime state included; a process without a model
    axis refuses the shards."""
    import os
    import socket
    import subprocess
    import sys

    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES="")
    tiny = ["--d-model", "32", "--n-layers", "2", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64",
            "--vocab-size", "300", "--n-slots", "4", "--d-slot", "16", "--d-k", "8", "--d-v", "8", "--screened-layers", "1",
            # a constant learning rate: the schedule depends on the planned number of steps, which differs between the legs
            "--lr-init", "0.001", "--lr-final", "0.001", "--warmup-steps", "0"]

    def launch(out, steps, *extra):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
               "127.0.0.1", "--master-port", str(port), "-m", "rwkv7m_b200.cli.train_binidx_distributed", "--steps",
               str(steps), "--mesh-axis-names", "data", "model", "--mesh-axis-sizes", "1", "2", "--param-axis-name", "model",
               "--collective-timeout-s", "60", "--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2",
               "--print-every", "0", "--output-dir", str(out), "--save-every", "2", "--device", "cpu",
               "--checkpoint-backend", "orbax", "--phase", "read_write", "--sampling-mode", "sequential", "--carry-state",
               *extra] + tiny
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=str(root))
        assert res.returncode == 0, res.stderr[-3000:]

    def losses(out):
        return [json.loads(l)["loss"] for l in (out / "metrics.jsonl").read_text().splitlines() if '"train"' in l]

    whole, split = tmp_path / "whole", tmp_path / "split"
    launch(whole, 4)
    launch(split, 2)
    ckpt = split / "ckpt-00000002"
    names = sorted(p.name for p in ckpt.iterdir())
    assert "tp_state.rank00000.safetensors" in names and "tp_state.rank00001.safetensors" in names
    assert "model.safetensors" in names and "runtime_state.rank00001.safetensors" in names
    payload = json.loads((ckpt / "checkpoint.json").read_text())
    assert payload["backend"] == "sharded" and payload["layout"] == "tensor_parallel" and payload["model_parallel"] == 2
    launch(split, 2, "--resume", str(ckpt))
    assert losses(split) == pytest.approx(losses(whole), rel=1e-5)
    # the gathered model file is the exchange artifact: a plain runtime loads it
    import rwkv7m_b200 as R

    params, config, _ = R.load_model_safetensors(ckpt / "model.safetensors")
    rt = R.load_runtime_params(R.create_runtime(0, config, batch_size=1), params)
    logits, _ = R.infer_prefill(rt, torch.tensor([[1, 2, 3, 4]], dtype=torch.int32))
    assert torch.isfinite(logits).all()
    # one process without a model axis cannot take the shards
    argv = ["--steps", "1", "--resume", str(ckpt), "--data-file", tiny_binidx, "--ctx-len", "4", "--global-batch-size", "2",
            "--print-every", "0", "--output-dir", str(tmp_path / "alone"), "--device", "cpu"] + tiny
    with pytest.raises(ValueError, match="tensor-parallel shards"):
        train_binidx_distributed.run_distributed_training(train_binidx_distributed.parse_args(argv))


def test_comparison_matrix_profiles_seeds_provenance_and_tables(tiny_binidx, tmp_path, capsys):
    """``rwkv7m-compare-variants matrix``: what the reference's wrapper scripts do (scripts/compare_minipile.sh,
    comparison.sh:925-1245): a size profile with overrides, one run directory per seed with ``parameters.env``,
    ``protocol.md``, replayable ``commands.sh`` and ``parameter_counts.csv``; ``--no-run`` stops there; a real run adds the
    three summary tables, the core-parity report and the cross-seed aggregate."""
    from rwkv7m_b200.cli import compare_matrix, compare_variants

    assert compare_matrix.PROFILES["small"]["d_model"] == 768 and compare_matrix.PROFILES["smoke"]["steps"] == 50
    tiny = ["--d-model", "32", "--n-heads", "2", "--head-size", "16", "--d-ffn", "64", "--n-layers", "2", "--d-slot", "16",
            "--d-k", "8", "--d-v", "8", "--n-slots", "4", "--device", "cpu"]
    # 1. dry run of the full-size plan: nothing is trained, the provenance files and exact parameter counts exist
    root = tmp_path / "plan_only"
    assert compare_variants.main(["matrix", "--profile", "smoke", "--no-run", "--root", str(root), "--run-id", "dry",
                                  "--seeds", "7"]) == 0
    run = root / "dry-seed7"
    assert {p.name for p in run.iterdir()} == {"parameters.env", "protocol.md", "commands.sh", "parameter_counts.csv"}
    env = dict(l.split("=", 1) for l in (run / "parameters.env").read_text().splitlines())
    assert env["PROFILE"] == "smoke" and env["SEED"] == "7" and "--d-model 256" in env["TRAINER_FLAGS"]
    commands = (run / "commands.sh").read_text()
    assert commands.count("rwkv7m-train-binidx-dp") == 4 and "--no-screening" in commands and os.access(run / "commands.sh", os.X_OK)
    counts = {r["variant"]: int(r["trainable_params"]) for r in csv.DictReader(open(run / "parameter_counts.csv"))}
    assert counts["local_param_control"] >= counts["local_mechanism"] > counts["local_core_baseline"]
    capsys.readouterr()

    # 2. two seeds of a tiny model, with the core-parity check
    root = tmp_path / "runs"
    argv = ["matrix", "--profile", "smoke", "--seeds", "1", "2", "--root", str(root), "--run-id", "t", "--data-file", tiny_binidx,
            "--steps", "3", "--ctx-len", "4", "--global-batch-size", "2", "--vocab-size", "300", "--eval-every", "1",
            "--eval-steps", "1", "--screened-layers", "1", "--loss-targets", "100", "--verify-core-parity"] + tiny
    assert compare_variants.main(argv) == 0
    capsys.readouterr()
    for seed in (1, 2):
        run = root / f"t-seed{seed}"
        names = {p.name for p in run.iterdir()}
        assert {"local_metric_summary.csv", "learning_speed_summary.csv", "learning_target_hits.csv", "summary.json",
                "upstream_core_parity", *compare_variants.VARIANT_ORDER} <= names
        assert json.loads((run / "upstream_core_parity" / "parity_report.json").read_text())["passed"] is True
        rows = list(csv.DictReader(open(run / "local_metric_summary.csv")))
        assert [r["variant"] for r in rows] == list(compare_variants.VARIANT_ORDER)
        assert all(int(r["train_steps"]) == 3 and int(r["tokens_seen"]) == 3 * 8 and float(r["final_eval_loss"]) > 0 for r in rows)
        speed = list(csv.DictReader(open(run / "learning_speed_summary.csv")))
        assert all(float(r["best_eval_loss"]) <= float(r["final_eval_loss"]) + 1e-9 and float(r["eval_loss_auc_mean"]) > 0 for r in speed)
        hits = list(csv.DictReader(open(run / "learning_target_hits.csv")))
        assert {h["target"] for h in hits} >= {"100", "local_core_baseline_final", "local_param_control_final"}
        assert all(h["hit"] == "1" and int(h["hit_step"]) >= 1 for h in hits if h["target"] == "100")
    agg = list(csv.DictReader(open(root / "seed_aggregate.csv")))
    row = next(r for r in agg if r["variant"] == "local_mechanism" and r["metric"] == "final_eval_loss")
    assert row["n_seeds"] == "2" and float(row["std"]) >= 0 and float(row["mean"]) > 0
    # the other sub-commands still hand trainer flags through untouched
    plan = compare_variants.plan_variants(["--vocab-size", "300", "--screened-layers", "1"] + tiny)
    assert plan["variants"]["local_mechanism"]["trainable_params"] > plan["variants"]["local_core_baseline"]["trainable_params"]


def test_evaluation_tool_on_a_model_axis_matches_one_process(tiny_binidx, tmp_path):
    """``rwkv7m-eval-binidx --model-axis-size 2`` under a two-process launcher (each process holds half of the projections)
    reports the loss that one process reports for the same checkpoint and batches."""
    import socket
    import subprocess
    import sys

    out = tmp_path / "run"
    tiny = ["--vocab-size", "300", "--d-model", "32", "--d-ffn", "64", "--n-layers", "2", "--n-heads", "2", "--head-size", "16",
            "--no-screening", "--device", "cpu"]
    args = train_binidx.parse_args(["--data-file", tiny_binidx, "--ctx-len", "4", "--steps", "2", "--print-every", "0",
                                    "--output-dir", str(out)] + tiny)
    _, _, ckpt = train_binidx.run_training(args)
    base = ["--data-file", tiny_binidx, "--checkpoint", str(ckpt), "--ctx-len", "4", "--batch-size", "2", "--steps", "3",
            "--print-every", "0", "--device", "cpu"]
    single = eval_binidx.evaluate_binidx(eval_binidx.parse_args(base))
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    root = Path(__file__).resolve().parents[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), "-m", "rwkv7m_b200.cli.eval_binidx", "--model-axis-size", "2"] + base
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(root),
                         env=dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("eval tokens=")]
    assert len(lines) == 1                                        # only the first process reports
    loss = float(lines[0].split("loss=")[1].split()[0])
    assert loss == pytest.approx(single["loss"], rel=1e-4) and f"tokens={single['tokens']}" in lines[0]
    # the same rows with every sequence split along time over the two processes (whole model on each, state handed over)
    cmd = cmd[:cmd.index("--model-axis-size")] + ["--context-parallel-size", "2", "--carry-state", "--sampling-mode", "sequential"] + base
    cmd[cmd.index("--master-port") + 1] = str(port + 1 if port < 65000 else port - 1)
    carried = eval_binidx.evaluate_binidx(eval_binidx.parse_args(base + ["--carry-state", "--sampling-mode", "sequential"]))
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=str(root),
                         env=dict(os.environ, PYTHONPATH=str(root), CUDA_VISIBLE_DEVICES=""))
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [l for l in res.stdout.splitlines() if l.startswith("eval tokens=")]
    assert len(lines) == 1 and f"tokens={carried['tokens']}" in lines[0]
    assert float(lines[0].split("loss=")[1].split()[0]) == pytest.approx(carried["loss"], rel=1e-5)
