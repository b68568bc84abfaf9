"""Sphere ray tracer, 1024x768: four spheres, two lights, diffuse + specular shading, background looked up by ray
direction (reference: examples/notebooks/RayTracing.ipynb, cells 16-29). One thread per pixel, scene in constant
memory, output a float RGB device buffer (optionally written as a PPM file). The notebook's matplotlib display is
dropped: no graphics stack exists here. Oracle and timed CPU baseline: the same arithmetic in numpy."""
from __future__ import annotations

import ctypes
import sys
import time

import numpy as np
import torch

from ._lib import Light, Scene, Sphere, lib, ptr, stream, time_cuda

W, H = 1024, 768
SHINY_YELLOW = (0.95, 0.95, 0.4, 0.7, 0.6, 30.0)
GREEN_RUBBER = (0.3, 0.7, 0.3, 0.9, 0.1, 1.0)
SPHERES = [((-3, 0, -16), 2, SHINY_YELLOW), ((-1.0, -1.5, -12), 1.8, GREEN_RUBBER), ((1.5, -0.5, -18), 3, GREEN_RUBBER),
           ((7, 5, -18), 4, SHINY_YELLOW)]
LIGHTS = [((-20, 20, 20), 1.0), ((20, -20, 20), 0.5)]


def scene() -> Scene:
    s = Scene()
    s.n_spheres, s.n_lights = len(SPHERES), len(LIGHTS)
    for i, (c, r, m) in enumerate(SPHERES):
        s.spheres[i] = Sphere(*c, r, *m)
    for i, (p, inten) in enumerate(LIGHTS):
        s.lights[i] = Light(*p, inten)
    return s


def background(h: int = 256, w: int = 512) -> np.ndarray:
    """Procedural stand-in for the notebook's background.png: a vertical sky gradient."""
    t = np.linspace(0, 1, h, dtype=np.float32)[:, None, None]
    return np.broadcast_to((1 - t) * np.array([0.2, 0.4, 0.8], np.float32) + t * np.array([0.9, 0.9, 1.0], np.float32), (h, w, 3)).copy()


def render_gpu(bg: torch.Tensor | None) -> torch.Tensor:
    img = torch.empty(H, W, 3, dtype=torch.float32, device="cuda")
    sc = scene()
    bgp = ptr(bg) if bg is not None else ctypes.c_void_p(0)
    bh, bw = (bg.shape[0], bg.shape[1]) if bg is not None else (0, 0)
    assert lib().b2_ex_raytrace(ptr(img), bgp, H, W, bh, bw, ctypes.byref(sc), stream()) == 0
    return img


def render_cpu(bg: np.ndarray | None) -> np.ndarray:
    f = np.float32
    rows, cols = np.arange(H, dtype=f)[:, None], np.arange(W, dtype=f)[None, :]
    y = np.broadcast_to(-((f(2) * rows + 1) / f(H) - 1), (H, W))
    x = np.broadcast_to(((f(2) * cols + 1) / f(W) - 1) * f(W) / f(H), (H, W))
    d = np.stack([x, y, -np.ones_like(x)], -1)
    d = d / np.linalg.norm(d, axis=-1, keepdims=True)
    best = np.full((H, W), np.inf, f)
    hit = np.full((H, W), -1)
    for i, (c, r, _) in enumerate(SPHERES):
        L = -np.array(c, f)
        a = (d * d).sum(-1); b = 2 * (d @ L); cc = f(L @ L - r * r)
        disc = b * b - 4 * a * cc
        ok = disc >= 0
        sq = np.sqrt(np.where(ok, disc, 0))
        q = np.where(b > 0, -0.5 * (b + sq), -0.5 * (b - sq))
        with np.errstate(divide="ignore", invalid="ignore"):
            t0, t1 = q / a, cc / q
        t0 = np.where(t0 > t1, t1, t0)
        t0 = np.where(t0 < 0, t1, t0)
        ok &= t0 >= 0
        better = ok & (t0 < best)
        best = np.where(better, t0, best); hit = np.where(better, i, hit)
    out = np.zeros((H, W, 3), f)
    if bg is not None:
        bc = ((1 + d[..., 0]) * 0.5 * (bg.shape[1] - 1)).astype(int); br = ((1 + d[..., 1]) * 0.5 * (bg.shape[0] - 1)).astype(int)
        out[:] = bg[br, bc]
    else:
        out[:] = 0.02
    for i, (c, r, m) in enumerate(SPHERES):
        mask = hit == i
        if not mask.any():
            continue
        point = d[mask] * best[mask][:, None]
        Nn = point - np.array(c, f)
        Nn /= np.linalg.norm(Nn, axis=-1, keepdims=True)
        diff = np.zeros(len(point), f); spec = np.zeros(len(point), f)
        for p, inten in LIGHTS:
            ld = np.array(p, f) - point
            ld /= np.linalg.norm(ld, axis=-1, keepdims=True)
            diff += inten * np.maximum((ld * Nn).sum(-1), 0)
            I = -ld
            refl = I - Nn * ((I * Nn).sum(-1, keepdims=True) * 2)
            spec += np.power(np.maximum(-(refl * d[mask]).sum(-1), 0), m[5]) * inten
        res = np.array(m[:3], f) * (diff * m[3])[:, None] + (spec * m[4])[:, None]
        mx = res.max(-1, keepdims=True)
        out[mask] = np.where(mx > 1, res / mx, res)
    return out


def write_ppm(path: str, img: np.ndarray) -> None:
    data = (np.clip(img, 0, 1) * 255).astype(np.uint8)
    with open(path, "wb") as f:
        f.write(f"P6 {img.shape[1]} {img.shape[0]} 255\n".encode())
        f.write(data.tobytes())


def main() -> None:
    bg = background()
    t0 = time.perf_counter()
    want = render_cpu(bg)
    cpu_ms = (time.perf_counter() - t0) * 1e3
    bgd = torch.from_numpy(bg).cuda()
    got = render_gpu(bgd).cpu().numpy()
    bad = (np.abs(got - want).max(-1) > 2e-2).mean()
    assert bad < 2e-3, f"{bad:.4%} of pixels differ"      # silhouette pixels may flip between fp32 orderings
    ms = time_cuda(lambda: render_gpu(bgd))
    print(f"ray tracer {W}x{H}: CPU numpy {cpu_ms:.1f} ms, GPU {ms * 1e3:.1f} us ({cpu_ms / ms:.0f}x)")
    if len(sys.argv) > 1:
        write_ppm(sys.argv[1], got)


if __name__ == "__main__":
    main()
