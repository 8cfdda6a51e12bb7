"""Lloyd-Max calibration kernel (``omni_lloyd_max_fit``) against the reference-generated codebooks and the oracle.

The kernel forms cell means in fp64 and rounds once; the reference sums in fp32 in library order, so single
updates agree to an fp32 ulp or two (``STEP_ATOL``, checked over the first 30 iterations).  Over a full run the
iteration itself magnifies that: on the 409,600-sample groups of configuration 0 the reference is still moving
5e-5 per iteration when its 300-iteration cap stops it, and a last-bit difference at iteration 30 has grown to
2e-5 by iteration 100.  Full runs are therefore held to ``RUN_ATOL`` on the centroids and to an equal
quantisation error, and compared exactly wherever every cell mean is exact in both arithmetics.
"""
import pytest
import torch

import oracle as orc
from tests.helpers import load_golden, t, sha, config0_inputs

pytestmark = pytest.mark.gpu

STEP_ATOL = 1e-6     # centroids after a matched, small number of iterations (data of unit scale)
RUN_ATOL = 2e-4      # centroids after a full run (see the module docstring)


def mse(x, cb):
    x = x.double().reshape(-1, 1)
    return float((x - cb.double().reshape(1, -1)).abs().min(dim=1).values.pow(2).mean())


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def quant():
    from omnistack_rs_b200.quantization import codebook
    return codebook


def test_config0_codebooks_match_the_reference_fit(dev):
    """The eight per-head codebooks the reference fitted on the rotated keys of configuration 0."""
    g = load_golden("config0_codec.npz")
    K, _, _ = config0_inputs()
    if sha(K) != str(g["sha_K"]):
        pytest.skip("torch.randn stream differs from the one the fixtures were made with")
    Kr = orc.wht128(K)
    groups = [Kr[:, h].reshape(-1).to(dev) for h in range(8)]
    got = quant().calibrate_per_group(groups)
    assert got.shape == (8, 16) and got.dtype == torch.float32 and got.is_cuda
    gold = t(g["codebooks"])
    assert (got.cpu() - gold).abs().max() <= RUN_ATOL
    for h in (0, 5):
        assert abs(mse(groups[h], got[h]) / mse(groups[h], gold[h].to(dev)) - 1.0) <= 1e-6
    # matched short runs stay within rounding of the reference's algorithm
    short = quant().calibrate_per_group(groups[:2], max_iters=30).cpu()
    want = orc.lloyd_max_per_group([Kr[:, h].reshape(-1) for h in range(2)], max_iters=30)
    assert (short - want).abs().max() <= STEP_ATOL
    # host-resident samples take the same kernel and come back on the host
    one = quant().LloydMaxCalibrator().fit(Kr[:, 3].reshape(-1)).codebook
    assert one.device.type == "cpu" and torch.equal(one, got[3].cpu())


@pytest.mark.parametrize("case", ["normal", "heavy_tail", "ragged_groups", "bf16"])
def test_fit_matches_oracle(dev, case):
    gen = torch.Generator().manual_seed({"normal": 1, "heavy_tail": 2, "ragged_groups": 3, "bf16": 4}[case])
    if case == "normal":
        groups = [torch.randn(20000, generator=gen)]
    elif case == "heavy_tail":
        x = torch.randn(30000, generator=gen)
        groups = [torch.where(torch.rand(30000, generator=gen) < 0.01, x * 10, x)]
    elif case == "ragged_groups":
        groups = [torch.randn(n, generator=gen) * s + m for n, s, m in ((16, 1.0, 0.0), (777, 0.2, 3.0), (12345, 5.0, -1.0))]
    else:
        groups = [torch.randn(8192, generator=gen).to(torch.bfloat16)]
    scale = torch.stack([x.float().abs().max() for x in groups]).clamp(min=1.0).unsqueeze(1)
    on_dev = [x.to(dev) for x in groups]
    for iters, atol in ((1, STEP_ATOL), (10, STEP_ATOL), (300, RUN_ATOL)):
        want = orc.lloyd_max_per_group(groups, max_iters=iters)
        got = quant().calibrate_per_group(on_dev, max_iters=iters).cpu()
        assert ((got - want).abs() / scale).max() <= atol, iters
        assert (got[:, 1:] >= got[:, :-1]).all()


def test_empty_cells_and_exact_means(dev):
    """Five distinct sample values leave most cells empty: those centroids must stay where the equal-mass
    initialisation put them, and every mean is exact in fp32 and fp64 alike, so the result is bit-equal."""
    vals = torch.tensor([-2.0, -0.5, 0.0, 0.25, 4.0])
    x = vals[torch.randint(0, 5, (4096,), generator=torch.Generator().manual_seed(5))]
    want = orc.lloyd_max_fit(x)
    got = quant().calibrate_codebook(x.to(dev)).cpu()
    assert torch.equal(got, want)
    const = torch.full((64,), 1.5)
    assert torch.equal(quant().calibrate_codebook(const.to(dev)).cpu(), torch.full((16,), 1.5))


def test_iteration_count_and_initialisation(dev):
    """Direct C call: zero iterations return the equal-mass means; the count of iterations run is reported."""
    from omnistack_rs_b200 import _lib
    lib = _lib.ensure_init(dev)
    x = torch.randn(50000, generator=torch.Generator().manual_seed(6))
    xs = x.sort().values
    init = torch.stack([xs[i * 3125:(i + 1) * 3125].double().mean() for i in range(16)]).float()
    srt = xs.to(dev)
    off = torch.tensor([0, x.numel()], dtype=torch.int64, device=dev)
    nbytes = lib.omni_lloyd_max_workspace_bytes(x.numel())
    ws = torch.empty(nbytes // 8, dtype=torch.float64, device=dev)
    out = torch.empty(1, 16, device=dev)
    iters = torch.full((1,), -1, dtype=torch.int32, device=dev)

    def run(max_iters, tol=1e-6):
        _lib.check(lib.omni_lloyd_max_fit(_lib.ptr(srt), x.numel(), _lib.ptr(off), 1, max_iters, tol, _lib.ptr(ws), nbytes,
                                          _lib.ptr(out), _lib.ptr(iters), _lib.stream_ptr(dev)))
        torch.cuda.synchronize(dev)
        return out[0].cpu().clone(), int(iters.item())

    cb0, n0 = run(0)
    assert n0 == 0 and torch.equal(cb0, init)
    cb7, n7 = run(7)
    assert n7 == 7 and (cb7 - orc.lloyd_max_fit(x, max_iters=7)).abs().max() <= STEP_ATOL
    cb, n = run(300)
    assert 7 < n <= 300
    with pytest.raises(ValueError):
        _lib.check(lib.omni_lloyd_max_fit(_lib.ptr(srt), x.numel(), _lib.ptr(off), 1, 300, 1e-6, _lib.ptr(ws), 64,
                                          _lib.ptr(out), None, _lib.stream_ptr(dev)))


def reference_update(x, cb):
    """One update of the reference's iteration (assignment by first-index argmin, cell means), in torch ops."""
    assign = (x.unsqueeze(1) - cb.unsqueeze(0)).abs().argmin(dim=1)
    sums = torch.zeros(16, dtype=torch.float64, device=x.device).index_add_(0, assign, x.double())
    cnt = torch.bincount(assign, minlength=16).double()
    return torch.where(cnt > 0, (sums / cnt.clamp(min=1)).float(), cb)


def test_large_sample_update_and_fixed_point(dev):
    """4 M samples (more than the oracle iterates in seconds).  Iteration k + 1 of the kernel must be the
    reference's update applied to its iteration k, and a run that is allowed to converge must end on a fixed
    point of that update."""
    x = torch.randn(1 << 22, generator=torch.Generator(device=dev).manual_seed(8), device=dev)
    cb300 = quant().calibrate_codebook(x, max_iters=300)
    cb301 = quant().calibrate_codebook(x, max_iters=301)
    assert (reference_update(x, cb300) - cb301).abs().max() <= STEP_ATOL
    cb = quant().calibrate_codebook(x, max_iters=20000)
    assert (reference_update(x, cb) - cb).abs().max() < 2e-6
    assert (cb[1:] > cb[:-1]).all()
    assert mse(x[: 1 << 18], cb) <= mse(x[: 1 << 18], cb300) * (1 + 1e-6)
