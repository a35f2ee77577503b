"""Single-GPU n-way reduction kernels against a plain PyTorch reference (fp32/fp64 math)."""
import pytest
import torch

from allreduce_over_mpi_b200.ops import launch_count, reduce_nway, reduce_nway_scaled

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rand(n, dtype, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.rand(n, generator=g, dtype=torch.float64) * 2 - 1
    if dtype == torch.bool:
        return (x > 0.6).to(DEV)
    if dtype.is_floating_point:
        return x.to(dtype).to(DEV)
    return (x * 100).to(dtype).to(DEV)


def ref_sum(ts):
    if ts[0].dtype == torch.bool:
        return torch.stack(ts).any(0)
    if ts[0].dtype.is_floating_point:
        acc = torch.zeros_like(ts[0], dtype=torch.float64 if ts[0].dtype == torch.float64 else torch.float32)
        for t in ts:
            acc += t.to(acc.dtype)
        return acc.to(ts[0].dtype)
    acc = torch.zeros_like(ts[0])
    for t in ts:
        acc += t  # wraps like the kernel
    return acc


@pytest.mark.parametrize("n", list(range(1, 21)) + [32])
def test_fanin_1_to_20_fp32(n):
    ts = [rand(100_003, torch.float32, k) for k in range(n)]
    before = launch_count()
    out = reduce_nway(ts)
    assert launch_count() > before
    want = torch.stack(ts).double().sum(0)
    assert torch.allclose(out.double(), want, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.uint8, torch.int8,
                                   torch.int16, torch.int32, torch.int64, torch.bool])
@pytest.mark.parametrize("n", [2, 3, 5, 8])
def test_dtypes_sum(dtype, n):
    ts = [rand(65_541, dtype, k) for k in range(n)]
    out = reduce_nway(ts)
    want = ref_sum(ts)
    if dtype in (torch.bfloat16, torch.float16):
        # kernel rounds once from an fp32 accumulator; so does the reference above
        assert torch.allclose(out.float(), want.float(), atol=1e-2 if dtype == torch.bfloat16 else 2e-3)
        exact = torch.stack(ts).double().sum(0)
        assert torch.allclose(out.double(), exact, atol=4e-2)
    elif dtype.is_floating_point:
        assert torch.allclose(out.double(), torch.stack(ts).double().sum(0), atol=1e-5)
    else:
        assert torch.equal(out, want)


@pytest.mark.parametrize("dtype", [torch.uint8, torch.int8, torch.int16, torch.int32, torch.int64])
def test_band(dtype):
    info = torch.iinfo(dtype)
    ts = [torch.randint(info.min, info.max, (40_001,), dtype=dtype, device=DEV) for _ in range(4)]
    out = reduce_nway(ts, op="band")
    assert torch.equal(out, ts[0] & ts[1] & ts[2] & ts[3])
    with pytest.raises(Exception, match="unsupported type"):
        reduce_nway([torch.rand(8, device=DEV)] * 2, op="band")


@pytest.mark.parametrize("length", [0, 1, 3, 4, 5, 255, 256, 257, 4099, 1 << 20])
def test_lengths_and_tails(length):
    ts = [rand(length, torch.float32, k) for k in range(3)]
    out = reduce_nway(ts)
    assert torch.allclose(out, ts[0] + ts[1] + ts[2], atol=1e-6)


@pytest.mark.parametrize("offsets", [(1, 1, 1, 1), (0, 1, 2, 3), (3, 0, 0, 0), (0, 0, 0, 1)])
def test_misaligned_bases(offsets):
    """Views that start off a 16-byte boundary take the scalar path; the result is the same."""
    n = 10_007
    base = [rand(n + 8, torch.float32, k) for k in range(3)]
    ts = [b[o:o + n] for b, o in zip(base, offsets)]
    out_base = torch.zeros(n + 8, device=DEV)
    out = out_base[offsets[3]:offsets[3] + n]
    reduce_nway(ts, out=out)
    assert torch.allclose(out, ts[0] + ts[1] + ts[2], atol=1e-6)
    assert out_base[:offsets[3]].abs().sum() == 0 and out_base[offsets[3] + n:].abs().sum() == 0


@pytest.mark.parametrize("variant", [2, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20, 21, 22, 23, 24])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_variants_agree(variant, dtype):
    for n in (1, 2, 4, 8, 9):
        ts = [rand((1 << 20) + 24, dtype, k) for k in range(n)]
        assert torch.equal(reduce_nway(ts, variant=variant), reduce_nway(ts, variant=1)), (variant, n)


def test_tma_variant_other_types_and_large_fanin():
    ts = [rand(300_000, torch.int32, k) for k in range(20)]
    assert torch.equal(reduce_nway(ts, variant=2), ref_sum(ts))
    ts = [rand(70_000, torch.float64, k) for k in range(32)]
    assert torch.allclose(reduce_nway(ts, variant=2), torch.stack(ts).sum(0), atol=1e-12)


def test_in_place_output():
    ts = [rand(50_000, torch.float32, k) for k in range(4)]
    want = ts[0] + ts[1] + ts[2] + ts[3]
    reduce_nway(ts, out=ts[0])
    assert torch.allclose(ts[0], want, atol=1e-6)


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16),
                                                (torch.bfloat16, torch.float32), (torch.float32, torch.float32)])
def test_scaled_cast(in_dtype, out_dtype):
    ts = [rand(33_333, in_dtype, k) for k in range(8)]
    out = reduce_nway_scaled(ts, scale=1 / 8, out_dtype=out_dtype)
    want = (torch.stack(ts).float().sum(0) / 8).to(out_dtype)
    assert out.dtype == out_dtype
    assert torch.allclose(out.float(), want.float(), atol=1e-2 if out_dtype == torch.bfloat16 else 1e-6)


def test_bad_arguments():
    with pytest.raises(ValueError):
        reduce_nway([])
    with pytest.raises(ValueError):
        reduce_nway([torch.rand(4, device=DEV)] * 33)
    with pytest.raises(ValueError):
        reduce_nway([torch.rand(4, device=DEV), torch.rand(5, device=DEV)])


# U * 1000 + LD * 100 + ST * 10 + T of the 32-byte-access kernels (csrc/kernels/reduce_nway_wide.cu)
WIDE = [1000, 1001, 1003, 1010, 1011, 1013, 1110, 1111, 2000, 2010, 2011, 2013, 2110, 2113, 24, 13]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [2, 3, 4, 8])
def test_wide_access_variants_match_the_default_kernels(dtype, n):
    """Every 256-bit configuration and the 16-byte kernels (variants 13 and 24) give the same bits (same summation
    order), for a length with a ragged tail; configurations that have no instantiation for a fan-in fall back silently."""
    ts = [rand(1_000_003, dtype, 40 + k) for k in range(n)]
    want = reduce_nway(ts)
    exact = torch.stack(ts).double().sum(0)
    assert torch.allclose(want.double(), exact, atol=1e-5 if dtype == torch.float32 else 4e-2)
    for v in WIDE:
        out = reduce_nway(ts, variant=v)
        assert torch.equal(out, want), (v, (out.float() - want.float()).abs().max().item())
    # a base that is 16- but not 32-byte aligned takes the 16-byte kernels
    off = [t[4:] if dtype == torch.float32 else t[8:] for t in ts]
    assert torch.equal(reduce_nway(off, variant=2011), reduce_nway(off))


def test_host_pipeline_reduces_prefixes_of_pinned_vectors():
    """Operands in pinned host memory, chunked through the device: several fan-ins over shared inputs, a length
    that is not a multiple of the chunk, two calls back to back on one pipeline."""
    from allreduce_over_mpi_b200.ops import HostReducePipeline
    n, length = 5, 300_007
    g = torch.Generator().manual_seed(5)
    hin = [(torch.rand(length, generator=g) * 2 - 1).pin_memory() for _ in range(n)]
    hout = [torch.empty(length).pin_memory() for _ in range(3)]
    pipe = HostReducePipeline(device=DEV, chunk_bytes=256 << 10, max_inputs=n, max_outputs=3)
    for _ in range(2):
        for h in hout:
            h.fill_(float("nan"))
        pipe.run(hin, [1, 3, 5], hout)
        torch.cuda.synchronize()
        for fan, h in zip([1, 3, 5], hout):
            want = torch.stack(hin[:fan]).double().sum(0)
            assert torch.allclose(h.double(), want, atol=1e-5), fan
        hin[0].add_(1.0)
    with pytest.raises(Exception):
        pipe.run(hin, [6], hout[:1])
    pipe.close()
