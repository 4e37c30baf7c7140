"""gnn_halo_push on one GPU: the "peers" are plain buffers of the same device, so the row
movement (grouping by destination, interleaved visiting order, own-row copy, scalar and
128-bit variants, ragged and empty groups) is checked without a second GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("width", [512, 47, 4, 1, 100])
@pytest.mark.parametrize("groups", [[0, 300, 0, 1, 77], [5], [0, 0], [1000, 3, 0, 0, 0, 0, 0, 250], [0]])
@pytest.mark.parametrize("with_own", [True, False])
def test_halo_push_rows(cuda, width, groups, with_own):
    from ae_mlsys_gnn_b200.peer import halo_push

    gen = torch.Generator().manual_seed(width * 131 + len(groups))
    n = 1200
    x = torch.randn(n, width, generator=gen).to(cuda)
    world = len(groups)
    send = [torch.randint(0, n, (c,), generator=gen, dtype=torch.int32) for c in groups]
    send_idx = torch.cat(send).to(cuda)
    offs = [0]
    for c in groups:
        offs.append(offs[-1] + c)
    # every "peer" buffer has a margin in front and behind that must stay untouched
    bufs = [torch.full((c + 2, width), -7.0, device=cuda) for c in groups]
    dst = [b[1:].data_ptr() if c else 0 for b, c in zip(bufs, groups)]
    n_own = 333 if with_own else 0
    own = torch.full((n_own + 2, width), -7.0, device=cuda)
    halo_push(x, send_idx, offs, dst, own[1:].data_ptr() if with_own else 0, n_own)
    torch.cuda.synchronize()
    for b, idx, c in zip(bufs, send, groups):
        assert torch.equal(b[1:1 + c], x[idx.to(cuda).long()])
        assert bool((b[0] == -7.0).all()) and bool((b[-1] == -7.0).all())
    if with_own:
        assert torch.equal(own[1:1 + n_own], x[:n_own])
    assert bool((own[0] == -7.0).all()) and bool((own[-1] == -7.0).all())


def test_halo_push_ranges(cuda):
    """Part of a send list per destination (what a block-wise producer pushes early): exactly the
    rows of the ranges arrive, at the start of the given destinations."""
    from ae_mlsys_gnn_b200.peer import halo_push_ranges

    gen = torch.Generator().manual_seed(5)
    n, width = 900, 128
    x = torch.randn(n, width, generator=gen).to(cuda)
    send_idx = torch.randint(0, n, (700,), generator=gen, dtype=torch.int32).to(cuda)
    begs, cnts = [10, 0, 300, 650], [90, 0, 200, 50]
    bufs = [torch.full((c + 2, width), -7.0, device=cuda) for c in cnts]
    dst = [b[1:].data_ptr() if c else 0 for b, c in zip(bufs, cnts)]
    halo_push_ranges(x, send_idx, begs, cnts, dst)
    torch.cuda.synchronize()
    for b, beg, c in zip(bufs, begs, cnts):
        assert torch.equal(b[1:1 + c], x[send_idx[beg: beg + c].long()])
        assert bool((b[0] == -7.0).all()) and bool((b[-1] == -7.0).all())
