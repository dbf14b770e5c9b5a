"""Parity of the framework's network against the independent upstream-layout x070 oracle, through the
capture -> archive -> verify CLIs; single-item binidx view; tensor-parallel audit."""

import json

import numpy as np
import pytest
import torch

from rwkv7m_b200.cli import audit_model_parallel, capture_upstream_reference, prepare_upstream_binidx, verify_upstream_rwkv7
from rwkv7m_b200.data.binidx import MMapIndexedDataset


def _archive(tmp_path, *extra):
    path = str(tmp_path / "ref.npz")
    assert capture_upstream_reference.main([path, "--d-model", "128", "--n-layers", "2", "--vocab-size", "384",
                                            "--tokens", "12", "--optimizer-step", *extra]) == 0
    return path


def test_capture_then_verify_passes_on_cpu_fp32(tmp_path):
    path = _archive(tmp_path, "--save-layers")
    out = tmp_path / "report.json"
    assert verify_upstream_rwkv7.main([path, "--device", "cpu", "--json-out", str(out)]) == 0
    rep = json.loads(out.read_text())
    assert rep["passed"] and rep["parameter_coverage"]["complete"]
    assert rep["logits"]["max_abs"] < 1e-4
    assert rep["gradients"]["global_cosine_similarity"] > 0.9999 and rep["gradients"]["global_relative_l2"] < 1e-3
    assert rep["optimizer_step"]["passed"]
    assert sorted(rep["parameter_coverage"]["ignored_names"]) == [f"blocks.0.att.v{i}" for i in range(3)]


def test_verify_detects_a_wrong_reference(tmp_path):
    path = _archive(tmp_path)
    data = dict(np.load(path))
    data["reference_logits"] = data["reference_logits"] + 0.5
    bad = str(tmp_path / "bad.npz")
    np.savez(bad, **data)
    assert verify_upstream_rwkv7.main([bad, "--device", "cpu"]) == 1
    # strict mode rejects tensors outside the mapping
    data = dict(np.load(path))
    data["weight::blocks.0.att.extra"] = np.zeros(3, dtype=np.float32)
    np.savez(bad, **data)
    assert verify_upstream_rwkv7.main([bad, "--device", "cpu"]) == 1


@pytest.mark.gpu
def test_cuda_bf16_model_matches_archive(tmp_path):
    path = _archive(tmp_path)
    rep = verify_upstream_rwkv7.verify_archive(path, dtype="bfloat16", device="cuda")
    assert rep["logits"]["passed"], rep["logits"]
    assert rep["gradients"]["global_cosine_similarity"] > 0.99, rep["gradients"]["global_cosine_similarity"]
    assert rep["optimizer_step"]["global_cosine_similarity"] > 0.9


def test_single_item_view_shares_the_bin(tiny_binidx, tmp_path):
    out = str(tmp_path / "view" / "single")
    n = prepare_upstream_binidx.prepare_single_item_view(tiny_binidx, out)
    src, view = MMapIndexedDataset(tiny_binidx), MMapIndexedDataset(out)
    assert len(view) == 1 and n == src.data_size == view.data_size
    np.testing.assert_array_equal(view.get(0, 0, n), src.get_global(0, n))
    assert prepare_upstream_binidx.prepare_single_item_view(tiny_binidx, out) == n  # idempotent


def test_model_parallel_audit_world_of_one():
    rep = audit_model_parallel.run_audit(audit_model_parallel.parse_args(["--cpu"]))
    assert rep["forward"]["finite"] and rep["train_step"]["finite"] and rep["train_step"]["optimizer_step"] == 1
    assert rep["contract"]["has_row_parallel_kernel"] and rep["contract"]["has_column_parallel_kernel"]
    assert rep["parameters"]["layers.0.block.att.output.weight"]["shard_dim"] == 1
    assert rep["forward"]["collectives"]["calls"]["all_gather_into_tensor"] >= 4


def test_convert_tool_round_trips_between_the_layouts(tmp_path):
    """``rwkv7m-convert-upstream``: a portable file exported to the upstream layout and imported again gives the same
    tensors and the same logits; the import infers the configuration from the shapes and reports full coverage; a model
    with screened layers is refused for export; an upstream file with a stray tensor fails unless allowed."""
    import json

    import rwkv7m_b200 as R
    from rwkv7m_b200.cli import convert_upstream

    cfg = R.tiny_config(vocab_size=300, d_model=32, n_layers=2, n_heads=2, head_size=16, use_screening=False)
    cfg.d_ffn = 64
    rt = R.create_runtime(0, cfg, batch_size=1)
    with torch.no_grad():      # the output projections start at zero: move them so that the logits depend on every tensor
        for p in rt.model.parameters():
            p.add_(torch.randn_like(p) * 0.02)
    src = tmp_path / "model.safetensors"
    R.save_model_safetensors(src, rt.model, cfg)
    assert convert_upstream.main(["export", str(src), str(tmp_path / "up.pth")]) == 0
    state = torch.load(tmp_path / "up.pth", weights_only=True)
    assert "emb.weight" in state and "blocks.1.att.key.weight" in state and state["blocks.0.att.v0"].abs().sum() == 0
    rc = convert_upstream.main(["import", str(tmp_path / "up.pth"), str(tmp_path / "back.safetensors"), "--head-size", "16",
                                "--dtype", "float32", "--report", str(tmp_path / "report.json")])
    assert rc == 0
    report = json.loads((tmp_path / "report.json").read_text())
    assert report["coverage"]["complete"] and report["spec"]["n_layers"] == 2 and report["spec"]["d_ffn"] == 64
    params, config, meta = R.load_model_safetensors(tmp_path / "back.safetensors")
    assert config.d_model == 32 and config.n_heads == 2 and not (config.use_screening and config.screening.screened_layers)
    other = R.load_runtime_params(R.create_runtime(7, config, batch_size=1), params)
    ids = torch.tensor([[1, 2, 3, 4, 5]], dtype=torch.int32)
    a, _ = R.infer_prefill(rt, ids)
    b, _ = R.infer_prefill(other, ids)
    assert torch.allclose(a, b, atol=1e-6)
    # the .safetensors flavour of the upstream layout, and a stray tensor
    assert convert_upstream.main(["export", str(src), str(tmp_path / "up.safetensors")]) == 0
    state["blocks.0.att.not_a_tensor"] = torch.zeros(3)
    torch.save(state, tmp_path / "stray.pth")
    with pytest.raises(ValueError, match="unexpected upstream tensors"):
        convert_upstream.main(["import", str(tmp_path / "stray.pth"), str(tmp_path / "x.safetensors"), "--head-size", "16"])
    assert convert_upstream.main(["import", str(tmp_path / "stray.pth"), str(tmp_path / "x.safetensors"), "--head-size", "16",
                                  "--allow-unexpected-weights"]) == 0
    screened = R.create_runtime(0, R.tiny_config(vocab_size=300, d_model=32, n_layers=2, n_heads=2, head_size=16), batch_size=1)
    R.save_model_safetensors(tmp_path / "screened.safetensors", screened.model, screened.config)
    with pytest.raises(ValueError, match="screening"):
        convert_upstream.main(["export", str(tmp_path / "screened.safetensors"), str(tmp_path / "no.pth")])
