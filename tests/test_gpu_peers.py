"""The peer-store epilogue of the attention kernels on one GPU: `peer_out` pointing at ordinary tensors of this GPU must
receive exactly what `out` receives, and `out=` must equal the tensor the plain call returns, bit for bit."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def unica():
    import unicaattention_b200 as unica

    return unica


def tensors(heads, n_queries, n_keys, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((1, heads, n_queries, 128), device="cuda", dtype=torch.bfloat16, generator=g)
    k, v = (torch.randn((1, heads, n_keys, 128), device="cuda", dtype=torch.bfloat16, generator=g) for _ in range(2))
    return q, k, v


@pytest.mark.parametrize("preset", ["per_channel", "per_token", "outliers", "fast"])
@pytest.mark.parametrize("n_queries,n_keys,peers", [(1000, 777, 2), (128, 64, 7), (333, 2048, 1)])
def test_peer_outputs_get_the_same_rows(unica, preset, n_queries, n_keys, peers):
    q, k, v = tensors(3, n_queries, n_keys)
    want = unica.attention(q, k, v, **unica.PRESETS[preset])
    # the output as heads 1..3 of a wider tensor: strides differ from q's, as in a sharded job
    wide = [torch.full((1, 5, n_queries, 128), 7.0, device="cuda", dtype=torch.bfloat16) for _ in range(peers + 1)]
    views = [w[:, 1:4] for w in wide]
    got = unica.attention(q, k, v, out=views[0], peer_out=[x.data_ptr() for x in views[1:]], **unica.PRESETS[preset])
    unica.check_status()
    assert got is views[0]
    for w in wide:
        assert torch.equal(w[:, 1:4], want)
        assert bool((w[:, 0] == 7).all()) and bool((w[:, 4] == 7).all())  # nothing outside the heads of the call


def test_peer_arguments_are_checked(unica):
    q, k, v = tensors(1, 128, 128)
    out = torch.empty_like(q)
    with pytest.raises(ValueError):
        unica.attention(q, k, v, peer_out=[out.data_ptr()])  # needs out
    with pytest.raises(ValueError):
        unica.attention(q, k, v, out=out, peer_out=[out.data_ptr()])  # a peer that is out itself
    with pytest.raises(ValueError):
        unica.attention(q, k, v, out=out, peer_out=[out.data_ptr() + 2])  # misaligned
    with pytest.raises(ValueError):
        unica.attention(q, k, v, out=out, peer_out=[out.data_ptr() + 16 * i for i in range(1, 9)])  # more than 7
    with pytest.raises(ValueError):
        unica.attention(q, k, v, out=out.float())
