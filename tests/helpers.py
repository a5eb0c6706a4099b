"""Shared tolerance checks for the parity tests."""
import torch

# bf16 / fp16: rel 2e-2, abs 1e-2 (the target's stated bar); fp32: rel 1e-5.
BF16_RTOL, BF16_ATOL = 2e-2, 1e-2
F32_RTOL = 1e-5


def error_stats(actual: torch.Tensor, expected: torch.Tensor):
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    diff = (a - e).abs()
    max_abs = diff.max().item() if diff.numel() else 0.0
    denom = e.abs().clamp_min(1e-6)
    mean_rel = (diff / denom).mean().item() if diff.numel() else 0.0
    return max_abs, mean_rel


def assert_parity(actual: torch.Tensor, expected: torch.Tensor, what: str = "", magnitude: torch.Tensor = None):
    """`magnitude`: optional tensor of operand magnitudes for sums that can cancel (a residual add): the
    relative tolerance then applies to max(|expected|, |magnitude|), because eager rounds the addends to the
    tensor dtype before adding and that rounding error does not shrink with the sum."""
    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    assert actual.dtype == expected.dtype, f"{what}: dtype {actual.dtype} vs {expected.dtype}"
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert torch.isfinite(a).all() or not torch.isfinite(e).all(), f"{what}: non-finite values in the result"
    if expected.dtype == torch.float32:
        scale = e.abs().max().item() if e.numel() else 1.0
        rtol, atol = F32_RTOL, F32_RTOL * max(scale, 1e-30)
        if e.numel():
            # both readings of "rel 1e-5" are shown: the bound applied here (error against the tensor's largest
            # magnitude) and the element-wise ratio, which is large wherever an element is close to zero
            d = (a - e).abs()
            print(f"{what}: fp32 max|diff|/max|ref| = {d.max().item() / max(scale, 1e-30):.3g}, "
                  f"element-wise max rel = {(d / e.abs().clamp_min(1e-30)).max().item():.3g} "
                  f"(median |ref| {e.abs().median().item():.3g})")
    else:
        rtol, atol = BF16_RTOL, BF16_ATOL
    ref_mag = e.abs() if magnitude is None else torch.maximum(e.abs(), magnitude.detach().float().cpu().abs())
    bad = (a - e).abs() > (atol + rtol * ref_mag)
    if bad.any():
        max_abs, mean_rel = error_stats(actual, expected)
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.numel()} elements outside rtol={rtol} atol={atol:.3g}; "
            f"max_abs={max_abs:.4g} mean_rel={mean_rel:.4g}; first at {idx}: got {a[tuple(idx)].item()} want {e[tuple(idx)].item()}"
        )


def assert_bit_exact(actual: torch.Tensor, expected: torch.Tensor, what: str = ""):
    assert actual.shape == expected.shape, f"{what}: shape {tuple(actual.shape)} vs {tuple(expected.shape)}"
    assert actual.dtype == expected.dtype, f"{what}: dtype"
    a, e = actual.detach().cpu().contiguous(), expected.detach().cpu().contiguous()
    if a.dtype.is_floating_point:  # compare bit patterns, so NaNs and signed zeros count too
        it = {2: torch.int16, 4: torch.int32, 8: torch.int64}[a.element_size()]
        a, e = a.view(it), e.view(it)
    assert torch.equal(a, e), f"{what}: results differ bitwise"


class LaunchCounter:
    """Counts the kernel-launching calls made into the C ABI while active (``with LaunchCounter() as c: ...; c.n``)."""

    def __enter__(self):
        from xpu_graph_b200 import lib

        self.n = 0
        self.names = []

        def before(name, args):
            if name not in lib.QUERY_ENTRY_POINTS:
                self.n += 1
                self.names.append(name)

        self._cm = lib.call_hook(before=before)
        self._cm.__enter__()
        return self

    def __exit__(self, *exc):
        return self._cm.__exit__(*exc)
