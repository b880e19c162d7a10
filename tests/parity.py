"""Error measures shared by the GPU parity tests.

The operators are specified to a relative Frobenius error of 1e-2 against an fp32-accumulated
product.  A norm over the whole output cannot see a few wrong rows or one wrong tile of a large
matrix, so the GEMM tests apply the same bound to every 128 x 256 output tile on its own and add a
loose element-wise bound."""
import torch

GEMM_TOL = 1e-2      # relative Frobenius error, whole output and per tile
GEMM_ABS_FACTOR = 8  # max-abs error allowed = this many times the largest 16-bit rounding step of the output


def tile_rel_errors(c: torch.Tensor, ref: torch.Tensor, tm: int = 128, tn: int = 256) -> torch.Tensor:
    """Relative Frobenius error of every ``tm x tn`` tile (ragged edges padded with zeros)."""
    c, ref = c.float(), ref.float().to(c.device)
    M, N = ref.shape
    pm, pn = (-M) % tm, (-N) % tn
    if pm or pn:
        c = torch.nn.functional.pad(c, (0, pn, 0, pm))
        ref = torch.nn.functional.pad(ref, (0, pn, 0, pm))
    gm, gn = c.shape[0] // tm, c.shape[1] // tn
    d = (c - ref).reshape(gm, tm, gn, tn).permute(0, 2, 1, 3).reshape(gm, gn, -1)
    r = ref.reshape(gm, tm, gn, tn).permute(0, 2, 1, 3).reshape(gm, gn, -1)
    return d.norm(dim=-1) / r.norm(dim=-1).clamp_min(1e-30)


def gemm_errors(c: torch.Tensor, ref: torch.Tensor):
    """``(global relative Frobenius, worst tile relative Frobenius, max-abs, max-abs allowed)``."""
    cf, rf = c.float(), ref.float().to(c.device)
    glob = ((cf - rf).norm() / rf.norm()).item()
    worst = tile_rel_errors(cf, rf).max().item()
    maxabs = (cf - rf).abs().max().item()
    eps = 2.0 ** -8 if c.dtype == torch.bfloat16 else 2.0 ** -11
    allowed = GEMM_ABS_FACTOR * eps * max(rf.abs().max().item(), 1e-30)
    return glob, worst, maxabs, allowed


def assert_gemm_close(c: torch.Tensor, ref: torch.Tensor, what: str = "") -> None:
    glob, worst, maxabs, allowed = gemm_errors(c, ref)
    assert glob < GEMM_TOL, f"{what}: relative Frobenius error {glob:.3e}"
    assert worst < GEMM_TOL, f"{what}: worst 128 x 256 tile has relative Frobenius error {worst:.3e}"
    assert maxabs <= allowed, f"{what}: max-abs error {maxabs:.3e} above {allowed:.3e}"
