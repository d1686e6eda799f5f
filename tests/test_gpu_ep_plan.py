"""The device-side planner of the expert-parallel step (flymoe_expert_counts, flymoe_ep_plan_direct)
against the host-side planner ``flydsl_b200.ep.plan_direct`` on synthetic rows-per-(rank, expert)
matrices for 1, 2, 4 and 8 ranks: integer work, compared bit for bit.  One GPU is enough: the planner
only reads the matrix, it does not talk to the other ranks."""
import numpy as np
import pytest
import torch

from flydsl_b200 import _lib
from flydsl_b200.ep import plan_direct

pytestmark = pytest.mark.gpu


def test_expert_counts_matches_bincount():
    lib = _lib.load()
    g = torch.Generator().manual_seed(3)
    for E, rows in ((8, 1), (256, 131072), (64, 777), (1024, 5000)):
        eids = torch.sort(torch.randint(0, E, (rows,), generator=g, dtype=torch.int32)).values
        if E == 64:
            eids = eids[eids != 5]                     # an expert without rows
        d = eids.cuda()
        nv = torch.tensor([d.numel(), 0], dtype=torch.int32, device="cuda")
        out = torch.full((E,), -1, dtype=torch.int64, device="cuda")
        _lib.check(lib.flymoe_expert_counts(d.data_ptr(), nv.data_ptr(), out.data_ptr(), E, d.numel() + 9,
                                            torch.cuda.current_stream().cuda_stream), "expert_counts")
        assert torch.equal(out.cpu(), torch.bincount(eids.long(), minlength=E))


@pytest.mark.parametrize("world,E,unit,skew", [(1, 16, 128, False), (2, 16, 128, True), (4, 256, 128, False),
                                               (8, 256, 128, True), (8, 256, 16, False), (2, 8, 32, True)])
def test_device_plan_matches_host_plan(world, E, unit, skew):
    lib = _lib.load()
    per = E // world
    g = np.random.default_rng(100 + world + E + unit)
    counts = g.integers(0, 400, size=(world, E)).astype(np.int64)
    if skew:
        counts[:, ::3] = 0                              # experts nobody routes to
        counts[:, 1] *= 20
    H = 512
    off_x, off_scale, off_back = 0, 1 << 20, 1 << 24
    peer_base = (np.arange(world, dtype=np.int64) + 1) * (1 << 40)
    for rank in sorted({0, world - 1, world // 2}):
        dp = plan_direct(counts, rank, per, unit)
        cap = (dp.max_padded_rows // unit + 3) * unit      # some room beyond every layout
        dev = "cuda"
        d_counts = torch.from_numpy(counts).to(dev)
        d_peer = torch.from_numpy(peer_base).to(dev)
        tab = torch.full((3, E), -1, dtype=torch.int64, device=dev)
        s_ids = torch.full((cap,), -7, dtype=torch.int32, device=dev)
        s_e = torch.full((cap // unit,), -7, dtype=torch.int32, device=dev)
        nv = torch.full((2,), -7, dtype=torch.int32, device=dev)
        row_dst = torch.full((cap,), -7, dtype=torch.int64, device=dev)
        ws = torch.zeros(int(lib.flymoe_ep_plan_workspace_elems(world, E)), dtype=torch.int32, device=dev)
        _lib.check(lib.flymoe_ep_plan_direct(
            d_counts.data_ptr(), d_peer.data_ptr(), off_x, off_scale, off_back, tab[0].data_ptr(), tab[1].data_ptr(),
            tab[2].data_ptr(), s_ids.data_ptr(), s_e.data_ptr(), nv.data_ptr(), row_dst.data_ptr(), ws.data_ptr(),
            ws.numel(), world, rank, E, unit, H, cap, torch.cuda.current_stream().cuda_stream), "ep_plan_direct")
        torch.cuda.synchronize()
        owner = np.arange(E) // per
        assert np.array_equal(tab[2].cpu().numpy(), dp.pos_base)
        assert np.array_equal(tab[0].cpu().numpy(), peer_base[owner] + off_x + dp.pos_base * H)
        assert np.array_equal(tab[1].cpu().numpy(), peer_base[owner] + off_scale + dp.pos_base * (H // 128) * 4)
        assert nv.cpu().tolist() == [dp.padded_rows, dp.padded_rows]
        # the receiver's layout, row by row, from the host plan's segments
        want_ids = np.full(cap, (1 << 24) | cap, dtype=np.int64)
        want_dst = np.zeros(cap, dtype=np.int64)
        pos = 0
        for ln, src, srow in zip(dp.seg_len, dp.seg_src, dp.seg_src_row):
            if src >= 0:
                r = np.arange(ln)
                want_ids[pos:pos + ln] = pos + r
                want_dst[pos:pos + ln] = peer_base[src] + off_back + (srow + r) * H * 2
            pos += ln
        assert pos == dp.padded_rows
        assert np.array_equal(s_ids.cpu().numpy().astype(np.int64), want_ids)
        assert np.array_equal(row_dst.cpu().numpy(), want_dst)
        nblk = dp.padded_rows // unit
        assert np.array_equal(s_e.cpu().numpy()[:nblk], dp.block_expert)
        assert int(s_e.max()) < per and int(s_e.min()) >= 0
