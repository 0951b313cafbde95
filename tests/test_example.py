"""The benchmark script: table formatting and parameter generation on CPU, one tiny run on the GPU."""
import pytest
import torch

from flexsae_b200 import example


def test_table_has_the_reference_layout():
    rows = {"torch TopK": {32: {"ms": 8.787, "gib": 2.92}, 64: {"ms": 11.746, "gib": 2.92}},
            "fused (sm_100a) TopK": {32: {"ms": 0.5, "gib": 1.0}, 64: {"ms": 0.75, "gib": 1.25}}}
    lines = example.format_table(rows, [32, 64]).split("\n")
    assert lines[0] == "| Decoder backend | K=32 (ms / GiB) | K=64 (ms / GiB) |"
    assert lines[1] == "| --- | --- | --- |"
    assert lines[2] == "| torch TopK | 8.787 / 2.92 | 11.746 / 2.92 |"
    assert lines[3] == "| fused (sm_100a) TopK | 0.500 / 1.00 | 0.750 / 1.25 |"


def test_parameters_follow_the_reference_script():
    p = example.make_parameters(8, 4, 32, 16, torch.bfloat16, torch.device("cpu"))
    assert p["indices"].dtype == torch.long and p["indices"].shape == (8, 4)
    assert int(p["indices"].min()) >= 0 and int(p["indices"].max()) < 32
    assert p["vals"].dtype == torch.float32 and bool((p["vals"] >= 0).all()) and p["vals"].requires_grad
    assert p["weight"].shape == (32, 16) and p["weight"].dtype == torch.bfloat16 and p["weight"].requires_grad
    assert p["bias"].requires_grad and not p["target"].requires_grad


def test_chunked_torch_loss_equals_the_whole_batch():
    torch.manual_seed(0)
    p = example.make_parameters(10, 4, 32, 16, torch.float32, torch.device("cpu"))
    whole = example._step(example.hierarchical_sae_loss, p)
    grads = [p[k].grad.clone() for k in ("weight", "vals", "bias")]
    example._drop_grads(p)
    parts = example._torch_step_chunked(example.hierarchical_sae_loss, p, 4)      # 4 + 4 + 2 rows
    assert torch.allclose(whole, parts, rtol=1e-6)
    for g, k in zip(grads, ("weight", "vals", "bias")):
        assert torch.allclose(g, p[k].grad, rtol=1e-5, atol=1e-7)


def test_needs_a_gpu():
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(SystemExit):
        example.main(["--iters", "1"])


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["hier", "topk"])
def test_tiny_run(kind, capsys):
    r = example.main(["--kind", kind, "--B", "64", "--K", "32", "--F", "4096", "--D", "256", "--iters", "3", "--warmup", "1",
                      "--torch-chunk", "48"])
    assert abs(r["loss_fused"] - r["loss_torch"]) <= 1e-4 * abs(r["loss_torch"])
    assert r["fused"]["ms"] > 0 and r["torch"]["ms"] > 0 and r["fused"]["gib"] > 0
    assert "speed-up" in capsys.readouterr().out
