"""Example programs: CPU parts here, kernels against their CPU restatements under the gpu marker."""
import numpy as np
import pytest


def test_nbody_energy_matches_reference_constants():
    from mojo_b200.examples.nbody import run

    e0, e1 = run(1000)
    assert abs(e0 - (-0.169075164)) < 1e-9      # initial energy of the standard five-body system
    assert abs(e1 - (-0.169087605)) < 1e-9      # after 1000 steps of dt 0.01


def test_life_cpu_rule_blinker():
    from mojo_b200.examples.life import evolve_cpu

    g = np.zeros((5, 5), np.uint8)
    g[2, 1:4] = 1
    n = evolve_cpu(g)
    assert n[1:4, 2].tolist() == [1, 1, 1] and n.sum() == 3 and np.array_equal(evolve_cpu(n), g)


@pytest.mark.gpu
def test_example_kernels_match_cpu_restatements():
    import torch

    from mojo_b200.examples import life, mandelbrot, matmul, raytrace, reduce

    got, want = mandelbrot.gpu().cpu().numpy(), mandelbrot.cpu()
    # fused multiply-adds on the device move a few boundary pixels of the chaotic recurrence by an iteration or more
    assert (got != want).mean() < 5e-3
    g = torch.Generator().manual_seed(0)
    a, b = torch.rand(100, 70, generator=g), torch.rand(70, 130, generator=g)
    for v in (0, 1):
        torch.testing.assert_close(matmul.gpu_variant(a.cuda(), b.cuda(), v).cpu(), a @ b, atol=1e-4, rtol=1e-4)
    x = torch.rand(1 << 21, generator=g)
    assert abs(reduce.gpu_sum(x.cuda()) - float(x.double().sum())) < 1e-6 * x.numel()
    grid = (np.random.default_rng(0).random((257, 130)) < 0.4).astype(np.uint8)
    assert np.array_equal(life.evolve_gpu(torch.from_numpy(grid).cuda()).cpu().numpy(), life.evolve_cpu(grid))
    bg = raytrace.background()
    img = raytrace.render_gpu(torch.from_numpy(bg).cuda()).cpu().numpy()
    assert (np.abs(img - raytrace.render_cpu(bg)).max(-1) > 2e-2).mean() < 2e-3


def test_example_runner_runs_host_examples_and_reports_the_rest(capsys):
    from mojo_b200.examples.__main__ import main

    import torch

    if torch.cuda.is_available():
        pytest.skip("covered by the gpu run of the same runner")
    assert main([]) == 0
    out = capsys.readouterr().out
    assert "== nbody" in out and "skipped (needs a CUDA device)" in out
    assert main(["nosuch"]) == 2


@pytest.mark.gpu
def test_example_runner_runs_everything_on_a_gpu():
    from mojo_b200.examples.__main__ import main

    assert main(["deviceinfo", "mandelbrot", "nbody", "life"]) == 0
