"""Decoupled look-back scan and first-occurrence relabel against the oracle (bit-exact)."""
import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def capi():
    from shmtensor_b200 import capi
    return capi


@pytest.mark.parametrize("n", [1, 2, 255, 256, 2047, 2048, 2049, 100_003, 3_000_001])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_scan_matches_cumsum(capi, n, dtype):
    g = torch.Generator(device="cuda").manual_seed(n)
    a = torch.randint(-1000, 1000, (n,), generator=g, device="cuda").to(dtype)
    inc, exc = a.clone(), a.clone()
    capi.thrust_scan(inc)
    capi.exclusive_scan_(exc)
    capi.check_async()          # the look-back's bounded waits all completed
    want = oracle.scan_inclusive(a.cpu().numpy())
    assert np.array_equal(inc.cpu().numpy(), want)
    assert np.array_equal(exc.cpu().numpy(), oracle.scan_exclusive(a.cpu().numpy()))


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_scan_tile_edges_views_and_many_tiles(capi, dtype):
    """Lengths around multiples of the 32 KB and 64 KB tiles, ragged tails shorter than 16 bytes,
    views that start off a 16-byte boundary, and enough tiles for every persistent CTA to loop."""
    item = 4 if dtype == torch.int32 else 8
    per32k = 32768 // item
    g = torch.Generator(device="cuda").manual_seed(77)
    big = torch.randint(-50, 50, (24_000_011,), generator=g, device="cuda").to(dtype)
    sizes = [4 * per32k - 1, 4 * per32k, 4 * per32k + 1, 5 * per32k + 3, 16 * per32k + per32k // 2 + 1,
             1000 * per32k + 7 if item == 4 else 700 * per32k + 1, big.numel()]
    for n in sizes:
        for off in (0, 1, 3, 4):
            src = big[off:off + n] if off + n <= big.numel() else big[off:]
            for fn, excl in ((capi.thrust_scan, False), (capi.exclusive_scan_, True)):
                work = big.clone()[off:off + src.numel()]      # a view: same alignment as src
                fn(work)
                want = torch.cumsum(src, 0, dtype=dtype)
                if excl:
                    want = want - src
                assert torch.equal(work, want), (n, off, excl)
    capi.check_async()
    assert capi.device_fault() == 0


@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_scan_large_inputs_through_the_cluster_kernel(capi, dtype):
    """From 32 MB on, whole 256 KB super-tiles go through the persistent cluster kernel and the
    rest through the ticketed one, which carries on from the last super-tile's sum: lengths at and
    around super-tile multiples, more super-tiles than resident clusters (every cluster loops),
    inclusive and exclusive, values that wrap in int32."""
    item = 4 if dtype == torch.int32 else 8
    per_super = (256 << 10) // item
    g = torch.Generator(device="cuda").manual_seed(123)
    n_max = 700 * per_super + 12_345
    big = torch.randint(-(2 ** 20), 2 ** 20, (n_max,), generator=g, device="cuda").to(dtype)
    for n in (128 * per_super, 128 * per_super + 1, 129 * per_super - 1, 300 * per_super + 5 * 4096 + 3, n_max):
        for fn, excl in ((capi.thrust_scan, False), (capi.exclusive_scan_, True)):
            work = big[:n].clone()
            fn(work)
            capi.check_async()
            want = torch.cumsum(big[:n], 0, dtype=dtype)
            if excl:
                want = want - big[:n]
            assert torch.equal(work, want), (n, excl)
    assert capi.device_fault() == 0


def test_scan_int32_wraps_like_the_oracle(capi):
    a = torch.full((5000,), 2**30, dtype=torch.int32, device="cuda")
    want = oracle.scan_inclusive(a.cpu().numpy())
    capi.thrust_scan(a)
    assert np.array_equal(a.cpu().numpy(), want)
    e = torch.empty(0, dtype=torch.int32, device="cuda")
    capi.thrust_scan(e)  # empty input is a no-op
    with pytest.raises(RuntimeError, match="int32 or int64"):
        capi.thrust_scan(torch.zeros(4, device="cuda"))


def test_relabel_golden_vector(capi):
    g = load_golden("relabel.json")
    for dt in (torch.int64, torch.int32):
        ins = [torch.tensor(x, dtype=dt, device="cuda") for x in g["inputs"]]
        uniq, rel = capi.tensor_relabel(ins)
        assert uniq.dtype == dt and uniq.cpu().tolist() == g["unique"]
        assert [r.cpu().tolist() for r in rel] == g["relabel"]
        assert all(r.dtype == dt for r in rel)


@pytest.mark.parametrize("sizes,hi", [((1,), 5), ((1000, 3000), 500), ((5, 0, 7), 4),
                                      ((70_000, 1_200_000), 2_400_000), ((300_000,), 10),
                                      ((2000,) * 9, 3000)])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_relabel_random_matches_oracle(capi, sizes, hi, dtype):
    rng = np.random.default_rng(sum(sizes) + hi)
    ins_n = [rng.integers(0, hi, size=s).astype(np.int64) for s in sizes]
    if dtype == torch.int64:
        ins_n = [x + (1 << 35) for x in ins_n]  # ids beyond 32 bits
    ins = [torch.from_numpy(x).to(dtype).cuda() for x in ins_n]
    uniq, rel = capi.tensor_relabel(ins)
    wu, wr = oracle.tensor_relabel([x.cpu().numpy() for x in ins])
    assert np.array_equal(uniq.cpu().numpy(), wu)
    assert len(rel) == len(sizes)
    for a, b in zip(rel, wr):
        assert np.array_equal(a.cpu().numpy(), b)


def test_relabel_ids_as_slots_and_hashed_ids_share_one_table(capi):
    """Inputs whose table is larger than the cache use the ids themselves as slots when they all fit
    the table, and hash them when one does not (a larger or a negative id); calls of both kinds,
    one after the other on one context, all match the oracle."""
    n, top = 1_500_000, (1 << 22) - 1  # 2^22 slots serve 1,500,000 ids
    rng = np.random.default_rng(9)
    dense = rng.integers(0, 300_000, size=n).astype(np.int64)
    cases = []
    for extra in (top, top + 1, -5, None, 1 << 40, top):
        x = dense.copy()
        rng.shuffle(x)
        if extra is not None:
            x[rng.integers(0, n)] = extra
        cases.append(x)
    for x in cases:
        uniq, (rel,) = capi.tensor_relabel([torch.from_numpy(x).cuda()])
        wu, (wr,) = oracle.tensor_relabel([x])
        assert np.array_equal(uniq.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wr)
    x32 = cases[0].astype(np.int32)
    uniq, rel = capi.tensor_relabel([torch.from_numpy(x32[:700_000]).cuda(), torch.from_numpy(x32[700_000:]).cuda()])
    wu, wr = oracle.tensor_relabel([x32[:700_000], x32[700_000:]])
    assert np.array_equal(uniq.cpu().numpy(), wu)
    assert all(np.array_equal(a.cpu().numpy(), b) for a, b in zip(rel, wr))
    # one int32 array of odd length (16-byte loads of the largest-id pass, then a tail), dense and not
    for extra in (None, -7):
        y = np.concatenate([x32, x32[:3]])
        if extra is not None:
            y[-2] = extra
        uniq, (rel,) = capi.tensor_relabel([torch.from_numpy(y).cuda()])
        wu, (wr,) = oracle.tensor_relabel([y])
        assert np.array_equal(uniq.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wr)
    capi.check_async()


@pytest.mark.parametrize("spread", [1, 1_000_003])
def test_relabel_five_million_ids(capi, spread):
    """Inputs of 4 M ids and more take the compact kernel with 4,096-element tiles (and, like every
    input whose table exceeds the cache, the largest-id pass): dense ids (ids as slots) and ids
    spread beyond the table (hashed), with a ragged last tile."""
    rng = np.random.default_rng(77)
    x = rng.integers(0, 2_000_000, size=5_000_123).astype(np.int64) * spread
    uniq, (rel,) = capi.tensor_relabel([torch.from_numpy(x).cuda()])
    wu, (wr,) = oracle.tensor_relabel([x])
    assert np.array_equal(uniq.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wr)
    # the table is clean afterwards: a small input right behind it
    y = x[:1000]
    uniq, (rel,) = capi.tensor_relabel([torch.from_numpy(y).cuda()])
    wu, (wr,) = oracle.tensor_relabel([y])
    assert np.array_equal(uniq.cpu().numpy(), wu) and np.array_equal(rel.cpu().numpy(), wr)
    capi.check_async()


def test_relabel_is_repeatable_and_idempotent(capi):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randint(0, 100_000, (500_000,), generator=g, device="cuda")
    u1, (r1,) = capi.tensor_relabel([x])
    u2, (r2,) = capi.tensor_relabel([x])
    assert torch.equal(u1, u2) and torch.equal(r1, r2)
    assert torch.equal(u1[r1], x)                       # relabel inverts through unique
    u3, (r3,) = capi.tensor_relabel([u1])               # unique ids relabel to 0..n-1
    assert torch.equal(u3, u1) and torch.equal(r3, torch.arange(u1.numel(), device="cuda"))


def test_relabel_errors(capi):
    with pytest.raises(RuntimeError):
        capi.tensor_relabel([])
    # mixed integer widths are promoted, as the reference's torch::cat does
    u, (a, b) = capi.tensor_relabel([torch.tensor([5, 7], dtype=torch.int64, device="cuda"),
                                     torch.tensor([7, 9], dtype=torch.int32, device="cuda")])
    assert u.dtype == torch.int64 and u.cpu().tolist() == [5, 7, 9]
    assert a.cpu().tolist() == [0, 1] and b.cpu().tolist() == [1, 2]
    with pytest.raises(RuntimeError, match="int32 or int64"):
        capi.tensor_relabel([torch.zeros(2, device="cuda")])
    e = torch.empty(0, dtype=torch.int64, device="cuda")
    u, (r,) = capi.tensor_relabel([e])
    assert u.numel() == 0 and r.numel() == 0


def test_lookback_wait_is_bounded_and_reported(capi):
    """A look-back whose predecessor never publishes gives up after its spin limit: the host
    gets SHMT_ERR_TIMEOUT, and the same context keeps working afterwards."""
    from shmtensor_b200 import _lib
    dev = torch.device("cuda", torch.cuda.current_device())
    ctx = capi._ctx(dev)
    rc = _lib.lib.shmt_debug_lookback_timeout(ctx, torch.cuda.current_stream().cuda_stream)
    assert rc == _lib.ERR_TIMEOUT and "bounded look-back wait ran out" in _lib.last_error()
    a = torch.arange(1, 10_001, dtype=torch.int64, device="cuda")
    capi.thrust_scan(a)
    capi.check_async()
    assert a[-1].item() == 50_005_000
    u, (r,) = capi.tensor_relabel([torch.tensor([7, 7, 3], device="cuda")])   # table was re-cleaned
    assert u.cpu().tolist() == [7, 3] and r.cpu().tolist() == [0, 0, 1]
