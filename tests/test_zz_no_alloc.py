"""sp_cuda_attention_paged_static — the attention entry point that allocates no device memory.

It must give exactly what sp_cuda_attention gives for the same inputs (same kernels, same split count), on two
calls in a row that share the library's fixed scratch array, whether this file runs alone or after the others."""
import numpy as np
import pytest

from sapient_b200 import _lib, ops

pytestmark = pytest.mark.gpu
KV_PAGE = 16
MAX_FLOATS = 1 << 20  # SP_ATTENTION_STATIC_MAX_FLOATS


def _paged_inputs(torch, q, k, v):
    """Device tensors laid out as the entry point documents: q rows [sq, H*hd], a one-slot fp16 page pool with an
    identity page table, and each row's (slot, position)."""
    H, sq, hd = q.shape
    Hkv, sk, _ = k.shape
    n_pages = (sk + KV_PAGE - 1) // KV_PAGE
    pool = np.zeros((n_pages, 2, Hkv, KV_PAGE, hd), dtype=np.float16)
    for s in range(sk):
        pool[s // KV_PAGE, 0, :, s % KV_PAGE, :] = k[:, s, :].astype(np.float16)
        pool[s // KV_PAGE, 1, :, s % KV_PAGE, :] = v[:, s, :].astype(np.float16)
    dev = "cuda:0"
    d = {
        "q": torch.from_numpy(np.ascontiguousarray(q.transpose(1, 0, 2)).reshape(sq, H * hd)).to(dev),
        "pool": torch.from_numpy(pool).to(dev),
        "pt": torch.arange(n_pages, dtype=torch.int32, device=dev),
        "slot": torch.zeros(sq, dtype=torch.int32, device=dev),
        "pos": torch.arange(sk - sq, sk, dtype=torch.int32, device=dev),
        "out": torch.full((sq, H * hd), float("nan"), dtype=torch.float32, device=dev),
    }
    return d, n_pages


def _static_attention(torch, q, k, v, n_splits):
    H, sq, hd = q.shape
    Hkv = k.shape[0]
    d, n_pages = _paged_inputs(torch, q, k, v)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    st = _lib.lib().sp_cuda_attention_paged_static(
        0, d["q"].data_ptr(), H * hd, d["out"].data_ptr(), H * hd, sq, H, Hkv, hd, d["slot"].data_ptr(), d["pos"].data_ptr(),
        d["pool"].data_ptr(), d["pt"].data_ptr(), n_pages, n_pages, 0, n_splits, None)
    _lib.check(st)
    torch.cuda.synchronize()
    # the call took no device memory (the driver's free-memory figure is unchanged; the very first call of a process
    # may load the module that holds the scratch array, so only a drop larger than that array would be an allocation)
    assert free_before - torch.cuda.mem_get_info()[0] <= (8 << 20), (free_before, torch.cuda.mem_get_info()[0])
    return d["out"].cpu().numpy().reshape(sq, H, hd).transpose(1, 0, 2)


def _rand(seed, H, Hkv, sq, sk, hd):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((H, sq, hd)).astype(np.float32), rng.standard_normal((Hkv, sk, hd)).astype(np.float32),
            rng.standard_normal((Hkv, sk, hd)).astype(np.float32))


def test_static_scratch_matches_allocating_entry_point_twice():
    import torch

    # sp_cuda_attention splits the keys 8 ways when sq <= 4; the second call is smaller than the first, so it
    # runs over scratch that still holds the first call's partials
    for seed, shape in ((1, (8, 2, 2, 150, 64)), (2, (4, 4, 1, 37, 128))):
        q, k, v = _rand(seed, *shape)
        want = ops.gqa_attention(q, k, v)
        got = _static_attention(torch, q, k, v, n_splits=8)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), shape


def test_static_scratch_single_split_and_prefill_shape():
    import torch

    q, k, v = _rand(3, 4, 2, 9, 40, 32)  # sq > 4: the allocating entry point uses one split
    want = ops.gqa_attention(q, k, v)
    got = _static_attention(torch, q, k, v, n_splits=1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_static_scratch_rejects_oversized_request():
    import torch

    H, Hkv, sq, sk, hd = 32, 8, 16, 64, 128
    n_splits = 32
    assert sq * H * n_splits * (hd + 2) > MAX_FLOATS
    q, k, v = _rand(4, H, Hkv, sq, sk, hd)
    with pytest.raises(_lib.SapientCudaError, match="static buffer"):
        _static_attention(torch, q, k, v, n_splits=n_splits)
