# SPDX-License-Identifier: Apache-2.0
"""CUDA kernels of the dynamics/data layers against their CPU twins."""
import pytest
import torch

from nvalchemi_toolkit_b200.dynamics import _ops
from nvalchemi_toolkit_b200.ops import buffer
from tests.helpers import random_batch

pytestmark = pytest.mark.gpu


def _pair(sizes=(5, 17, 9), dtype=torch.float32):
    b = random_batch(list(sizes), dtype=dtype)
    b["forces"] = torch.randn_like(b.positions)
    b["velocities"] = torch.randn_like(b.positions)
    return b, b.clone().cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_vv_and_langevin_match_cpu(dtype):
    c, g = _pair(dtype=dtype)
    dt = torch.tensor([0.05, 0.03, 0.07], dtype=dtype)
    kT = torch.full((3,), 0.025, dtype=dtype)
    fr = torch.full((3,), 0.2, dtype=dtype)
    for x, dev in ((c, "cpu"), (g, "cuda")):
        _ops.vv_position_update(x.positions, x.velocities, x.forces, x.atomic_masses, dt.to(dev), x.batch_idx)
        _ops.vv_velocity_finalize(x.velocities, x.forces, x.atomic_masses, dt.to(dev), x.batch_idx)
        _ops.langevin_half_step(x.positions, x.velocities, x.forces, x.atomic_masses, dt.to(dev), kT.to(dev), fr.to(dev), 11,
                                x.batch_idx)
    tol = 1e-5 if dtype == torch.float32 else 1e-12
    assert torch.allclose(g.positions.cpu(), c.positions, atol=tol, rtol=tol)
    assert torch.allclose(g.velocities.cpu(), c.velocities, atol=tol, rtol=tol)


def test_reductions_and_fire_match_cpu():
    c, g = _pair()
    ke_c = _ops.compute_kinetic_energy(c.velocities, c.atomic_masses, c.batch_idx, 3)
    ke_g = _ops.compute_kinetic_energy(g.velocities, g.atomic_masses, g.batch_idx, 3)
    assert torch.allclose(ke_g.cpu(), ke_c, rtol=1e-5)
    for mode in ("sum", "max", "min", "mean"):
        a = _ops._segmented(c.positions, c.batch_idx, 3, mode)
        b = _ops._segmented(g.positions, g.batch_idx, 3, mode)
        assert torch.allclose(b.cpu(), a, rtol=1e-5, atol=1e-6)
    from nvalchemi_toolkit_b200.dynamics import FIRE
    from nvalchemi_toolkit_b200.models import DemoModelWrapper

    model = DemoModelWrapper()
    fc, fg = FIRE(model, dt=0.1), FIRE(model, dt=0.1)
    for f, x in ((fc, c), (fg, g)):
        f._init_state(x)
        for _ in range(3):
            f.pre_update(x)
    assert torch.allclose(g.positions.cpu(), c.positions, atol=1e-5)
    assert torch.allclose(g.velocities.cpu(), c.velocities, atol=1e-5)
    assert torch.allclose(fg._state["dt"].cpu(), fc._state["dt"])


def test_buffer_primitives():
    starts = torch.tensor([3, 10, 0], device="cuda")
    lens = torch.tensor([2, 0, 4], device="cuda")
    assert buffer.expand_segments(starts, lens).tolist() == [3, 4, 0, 1, 2, 3]
    for dtype, width in ((torch.float32, 3), (torch.float64, 4), (torch.int64, 1), (torch.bool, 3), (torch.float32, 16)):
        src = (torch.rand(9, width, device="cuda") * 10).to(dtype)
        dst = torch.zeros(6, width, device="cuda", dtype=dtype)
        buffer.copy_rows(src, torch.tensor([8, 1, 4], device="cuda"), dst, torch.tensor([0, 5, 2], device="cuda"))
        assert torch.equal(dst[[0, 5, 2]], src[[8, 1, 4]]) and not dst[[1, 3, 4]].any()


@pytest.mark.gpu
@pytest.mark.parametrize("rows", [1, 130, 5000])
def test_fused_radial_mlp_matches_fp32_reference(rows):
    """8 -> 64 -> 64 -> 64 with SiLU, value rows and (value, d/dr) row pairs, against float64 PyTorch."""
    from nvalchemi_toolkit_b200.models.mace import native
    from nvalchemi_toolkit_b200.models.mace.model import SILU_NORM

    torch.manual_seed(rows)
    dev = "cuda"
    ws = [torch.randn(8, 64, device=dev) / 8 ** 0.5, torch.randn(64, 64, device=dev) / 8, torch.randn(64, 64, device=dev) / 8,
          torch.randn(64, 640, device=dev) / 8]
    ef = torch.randn(rows, 2, 8, device=dev)

    def ref(x, t):
        x, t = x.double(), t.double()
        for w in ws[:3]:
            z, zt = x @ w.double(), t @ w.double()
            s = torch.sigmoid(z)
            x, t = z * s * SILU_NORM, s * (1 + z * (1 - s)) * SILU_NORM * zt
        return x, t

    want_v, want_t = ref(ef[:, 0], ef[:, 1])
    got = native._hidden_fused(ws, ef, True)
    assert got is not None and got.shape == (rows, 2, 64)
    scale = float(want_v.abs().max())
    assert float((got[:, 0].double() - want_v).abs().max()) < 4e-3 * scale
    assert float((got[:, 1].double() - want_t).abs().max()) < 4e-3 * float(want_t.abs().max())
    val = native._hidden_fused(ws, ef[:, :1].contiguous(), False)
    assert float((val.double() - want_v).abs().max()) < 4e-3 * scale
    assert native.fused_error_status(torch.device(dev)) == 0
    # the first layer alone keeps fp32 accuracy thanks to the hi/lo split of inputs and weights
    one = native._hidden_fused([ws[0], torch.eye(64, device=dev), torch.eye(64, device=dev), ws[3]], ef[:, :1].contiguous(), False)
    z = ef[:, 0].double() @ ws[0].double()
    l1 = z * torch.sigmoid(z) * SILU_NORM
    for _ in range(2):  # the two identity layers still apply the activation (and tf32 rounding of their input)
        l1 = l1 * torch.sigmoid(l1) * SILU_NORM
    assert float((one.double() - l1).abs().max()) < 2e-3 * float(l1.abs().max())


@pytest.mark.gpu
def test_halo_pull_and_push_add_rows_single_device():
    """Row gather from / reduction into 'peer' buffers addressed through a pointer table (one device: the table points at
    two local buffers that stand in for two ranks)."""
    dev = "cuda"
    torch.manual_seed(0)
    a, b = torch.randn(10, 6, device=dev), torch.randn(8, 6, device=dev)
    ptrs = torch.tensor([a.data_ptr(), b.data_ptr()], dtype=torch.int64, device=dev)
    home_rank = torch.tensor([1, 0, 1, 1, 0], dtype=torch.int32, device=dev)
    home_row = torch.tensor([7, 2, 0, 7, 9], dtype=torch.int32, device=dev)
    dst = torch.zeros(9, 6, device=dev)
    shift = torch.arange(30, dtype=torch.float32, device=dev).reshape(5, 6)
    torch.ops.nvalchemi.halo_pull_rows(dst, 4, home_rank, home_row, shift, ptrs)
    want = torch.stack([b[7], a[2], b[0], b[7], a[9]]) + shift
    assert torch.equal(dst[4:], want) and float(dst[:4].abs().sum()) == 0
    a0, b0 = a.clone(), b.clone()
    src = torch.randn(9, 6, device=dev)
    torch.ops.nvalchemi.halo_push_add_rows(src, 4, home_rank, home_row, ptrs)
    a0[2] += src[5]
    a0[9] += src[8]
    b0[7] += src[4] + src[7]
    b0[0] += src[6]
    assert torch.allclose(a, a0, atol=1e-6) and torch.allclose(b, b0, atol=1e-6)


@pytest.mark.gpu
def test_csr_fill_kernel_matches_mask_gathers():
    """Neighbour matrix -> CSR edge arrays: the one-pass kernel against the boolean-mask formulation."""
    from nvalchemi_toolkit_b200.models.mace import native

    torch.manual_seed(0)
    n, k = 1000, 24
    num = torch.randint(0, k + 5, (n,), dtype=torch.int32, device="cuda")   # some counts overflow the matrix width
    nm = torch.randint(0, n, (n, k), dtype=torch.int32, device="cuda")
    sh = torch.randint(-1, 2, (n, k, 3), dtype=torch.int32, device="cuda")
    got = native.build_csr(nm, num, sh)
    ref = native.build_csr(nm.long(), num, sh)                               # int64 matrix takes the torch path
    assert got.num_edges == ref.num_edges and got.max_count == ref.max_count
    assert torch.equal(got.eptr, ref.eptr) and torch.equal(got.esend, ref.esend)
    assert torch.equal(got.erecv, ref.erecv) and torch.equal(got.eS, ref.eS)
    none = native.build_csr(nm, num, None)
    assert torch.equal(none.esend, ref.esend) and int(none.eS.abs().sum()) == 0


@pytest.mark.gpu
def test_grouped_gemm_matches_fp32_reference():
    """One grouped tcgen05 launch (column slices of a wide matrix times packed weight blocks, different K per group,
    optional accumulation) against the same products in float32 PyTorch."""
    from nvalchemi_toolkit_b200.ops import gemm

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    m, c = 1000, 128
    a = torch.randn(m, 9 * c, device=dev, generator=g)
    w_small = [torch.randn(c, c, device=dev, generator=g) for _ in range(2)]
    w_big = torch.randn(3 * c, c, device=dev, generator=g)
    packed, rows = gemm.pack_weights(w_small + [w_big])
    groups = [(0, c, rows[0], 0), (c, c, rows[1], c), (2 * c, c, rows[1], 2 * c), (3 * c, 3 * c, rows[2], 3 * c),
              (6 * c, 3 * c, rows[2], 4 * c)]
    out = torch.full((m, 5 * c), float("nan"), device=dev)
    gemm.grouped(a, packed, out, c, groups, alpha=0.5)
    ws = [w_small[0], w_small[1], w_small[1], w_big, w_big]
    ref = torch.cat([0.5 * (a[:, ac: ac + k].double() @ w.double()) for (ac, k, _, _), w in zip(groups, ws)], dim=1)
    scale = float(ref.abs().max())
    assert float((out.double() - ref).abs().max()) < 2e-3 * scale  # tf32 operands
    base = torch.randn(m, 5 * c, device=dev, generator=g)
    acc = base.clone()
    gemm.grouped(a, packed, acc, c, groups, alpha=0.5, accumulate=True)
    assert float((acc.double() - base.double() - ref).abs().max()) < 2e-3 * scale
    # narrow outputs (N = 64) and a strided destination
    w64 = [torch.randn(c, 64, device=dev, generator=g) for _ in range(3)]
    p64, r64 = gemm.pack_weights(w64)
    wide = torch.zeros(m, 4 * 64 + 8, device=dev)
    gemm.grouped(a, p64, wide[:, :4 * 64], 64, [(i * c, c, r64[i % 3], i * 64) for i in range(4)])
    ref64 = torch.cat([a[:, i * c: (i + 1) * c].double() @ w64[i % 3].double() for i in range(4)], dim=1)
    assert float((wide[:, :256].double() - ref64).abs().max()) < 2e-3 * float(ref64.abs().max())
    assert float(wide[:, 256:].abs().max()) == 0.0
    assert gemm.check_errors(a) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("width", [3, 8, 512])
def test_halo_kernels_against_index_ops_single_process(width):
    """The peer-memory halo kernels on ONE GPU: three buffers of this process stand for three ranks' arenas (the kernels only
    see pointer tables).  Pull = gather of the owners' rows (+ optional shift), push-add / pull-add = scatter-add of the
    holders' ghost rows into the owners' rows, `used` masks skip rows; all against plain index operations."""
    from nvalchemi_toolkit_b200.ops import _native
    from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

    assert _native.available()
    ops = torch.ops.nvalchemi
    dev = torch.device("cuda", 0)
    n_own, n_ghost, world = 200, 96, 3
    cap = n_own + n_ghost
    p2p = P2PContext.single_process(4 * cap * width * 2 + (1 << 16), dev, world)
    buf, ptrs = p2p.arena.alloc((cap, width))
    g = torch.Generator(device="cpu").manual_seed(width)
    arenas = []
    for r in range(world):  # fill every "rank's" copy of the buffer through its base pointer
        view = p2p.arena._bufs[r][p2p.arena.offset_of(buf): p2p.arena.offset_of(buf) + 4 * cap * width].view(torch.float32).reshape(cap, width)
        view.copy_(torch.randn(cap, width, generator=g))
        arenas.append(view)
    home_rank = torch.randint(1, world, (n_ghost,), generator=g).to(torch.int32).to(dev)
    home_row = torch.randperm(n_own, generator=g)[:n_ghost].to(torch.int32).to(dev)
    shift = torch.randn(n_ghost, width, generator=g).to(dev) if width == 3 else None
    used = (torch.rand(n_ghost, generator=g) < 0.7).to(torch.uint8).to(dev)
    before = [a.clone() for a in arenas]
    # pull: ghost row k of rank 0 <- row home_row[k] of rank home_rank[k]
    ops.halo_pull_rows(buf, n_own, home_rank, home_row, shift, ptrs, None)
    want = torch.stack([before[int(r)][int(j)] for r, j in zip(home_rank.tolist(), home_row.tolist())])
    want = want + shift if shift is not None else want
    assert torch.equal(arenas[0][n_own:], want) and torch.equal(arenas[0][:n_own], before[0][:n_own])
    arenas[0][n_own:].copy_(before[0][n_own:])
    ops.halo_pull_rows(buf, n_own, home_rank, home_row, shift, ptrs, used)
    m = used.bool()
    assert torch.equal(arenas[0][n_own:][m], want[m]) and torch.equal(arenas[0][n_own:][~m], before[0][n_own:][~m])
    # push-add: ghost rows of rank 0 are added into their owners' rows
    for a, b in zip(arenas, before):
        a.copy_(b)
    ops.halo_push_add_rows(buf, n_own, home_rank, home_row, ptrs, None)
    for r in range(1, world):
        sel = home_rank == r
        ref = before[r].clone().index_add_(0, home_row[sel].long(), before[0][n_own:][sel])
        assert torch.allclose(arenas[r], ref, atol=1e-6)
    # pull-add (the owner's view): rank 0 owns rows dst_row[k], whose copies sit on rank peer[k] at row peer_row[k]
    for a, b in zip(arenas, before):
        a.copy_(b)
    n_send = 80
    dst_row = torch.randint(0, n_own, (n_send,), generator=g).to(torch.int32).to(dev)
    peer = torch.randint(1, world, (n_send,), generator=g).to(torch.int32).to(dev)
    peer_row = (n_own + torch.randperm(n_ghost, generator=g)[:n_send]).to(torch.int32).to(dev)
    ops.halo_pull_add_rows(buf, dst_row, peer, peer_row, ptrs, None, None)
    copies = torch.stack([before[int(r)][int(j)] for r, j in zip(peer.tolist(), peer_row.tolist())])
    ref = before[0].clone().index_add_(0, dst_row.long(), copies)
    assert torch.allclose(arenas[0], ref, atol=1e-5)
    assert p2p.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("kick", [False, True])
def test_fused_force_return_and_half_kick_single_process(kick):
    """``halo_force_finalize``: owned gradient + the ghost copies' gradients on other (emulated) ranks -> force, and with a
    velocity array the closing half kick, against index operations; masked copies are skipped."""
    from nvalchemi_toolkit_b200.ops import _native
    from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext

    assert _native.available()
    ops = torch.ops.nvalchemi
    dev = torch.device("cuda", 0)
    n_own, n_ghost, world = 300, 120, 3
    cap = n_own + n_ghost
    p2p = P2PContext.single_process(4 * cap * 3 + n_ghost + (1 << 16), dev, world)
    gpos, ptrs = p2p.arena.alloc((cap, 3))
    used, used_ptrs = p2p.arena.alloc((n_ghost,), torch.uint8)
    g = torch.Generator().manual_seed(11)
    views, used_views = [], []
    for r in range(world):
        raw = p2p.arena._bufs[r]
        v = raw[p2p.arena.offset_of(gpos): p2p.arena.offset_of(gpos) + 4 * cap * 3].view(torch.float32).reshape(cap, 3)
        v.copy_(torch.randn(cap, 3, generator=g))
        u = raw[p2p.arena.offset_of(used): p2p.arena.offset_of(used) + n_ghost]
        u.copy_((torch.rand(n_ghost, generator=g) < 0.75).to(torch.uint8))
        views.append(v)
        used_views.append(u)
    # every third owned row has one or two copies on the other "ranks"
    rows, peers, prow = [], [], []
    for i in range(0, n_own, 3):
        for c in range(1 + (i % 2)):
            rows.append(i)
            peers.append(1 + (i + c) % (world - 1))
            prow.append(int(torch.randint(0, n_ghost, (1,), generator=g)))
    rows_t = torch.tensor(rows)
    copy_ptr = torch.zeros(n_own + 1, dtype=torch.int32)
    copy_ptr[1:] = torch.cumsum(torch.bincount(rows_t, minlength=n_own), 0)
    copy_peer = torch.tensor(peers, dtype=torch.int32, device=dev)
    copy_used_index = torch.tensor(prow, dtype=torch.int32, device=dev)
    copy_row = (copy_used_index + n_own).contiguous()
    forces = torch.empty(n_own, 3, device=dev)
    vel0 = torch.randn(n_own, 3, generator=g).to(dev)
    vel = vel0.clone()
    mass = (1.0 + torch.rand(n_own, generator=g)).to(dev)
    dt = torch.tensor([0.37], device=dev)
    bidx = torch.zeros(n_own, dtype=torch.int32, device=dev)
    extra = (vel, mass, dt, bidx) if kick else (None, None, None, None)
    ops.halo_force_finalize(gpos, copy_ptr.to(dev), copy_peer, copy_row, copy_used_index, ptrs, used_ptrs, forces, *extra)
    want = views[0][:n_own].clone()
    for i, p, j in zip(rows, peers, prow):
        if int(used_views[p][j]):
            want[i] += views[p][n_own + j]
    assert torch.allclose(forces, -want, atol=1e-6)
    if kick:
        assert torch.allclose(vel, vel0 + 0.5 * dt * (-want) / mass[:, None], atol=1e-6)
    else:
        assert torch.equal(vel, vel0)


@pytest.mark.gpu
def test_neighbor_build_fetches_ghost_positions_itself():
    """``ghost_pull``: the first kernel of the neighbour build loads the ghost rows from their owners' buffers (here two
    local buffers behind a pointer table), adds the image shift and stores them; rows, counts and shifts equal those of a
    separate pull followed by the plain build."""
    from nvalchemi_toolkit_b200 import neighbors as nb

    dev = "cuda"
    g = torch.Generator().manual_seed(5)
    box = 12.0
    n_own, n_ghost = 700, 260
    own = (torch.rand(n_own, 3, generator=g) * torch.tensor([box / 2, box, box])).to(dev)
    other = (torch.rand(900, 3, generator=g) * torch.tensor([box / 2, box, box]) + torch.tensor([box / 2, 0, 0])).to(dev)
    ptrs = torch.tensor([own.data_ptr(), other.data_ptr()], dtype=torch.int64, device=dev)
    home_rank = torch.ones(n_ghost, dtype=torch.int32, device=dev)
    home_row = torch.randperm(900, generator=g)[:n_ghost].to(torch.int32).to(dev)
    shift = torch.zeros(n_ghost, 3, device=dev)
    shift[::2, 0] = -box  # every other ghost is the periodic image on the far side
    cell = (torch.eye(3, device=dev) * box).reshape(1, 3, 3)
    pbc = torch.zeros(1, 3, dtype=torch.bool, device=dev)
    n = n_own + n_ghost
    bidx = torch.zeros(n, dtype=torch.int32, device=dev)
    bptr = torch.tensor([0, n], dtype=torch.int32, device=dev)
    ref = torch.zeros(n, 3, device=dev)
    ref[:n_own] = own
    torch.ops.nvalchemi.halo_pull_rows(ref, n_own, home_rank, home_row, shift, ptrs)
    want = nb.neighbor_matrix(ref, cell, pbc, bidx, bptr, 3.0, 96, num_rows=n_own)
    got_pos = torch.full((n, 3), float("nan"), device=dev)
    got_pos[:n_own] = own
    got = nb.neighbor_matrix(got_pos, cell, pbc, bidx, bptr, 3.0, 96, num_rows=n_own,
                             ghost_pull=(n_own, home_rank, home_row, shift, ptrs))
    assert torch.equal(got_pos, ref)
    assert torch.equal(got[1][:n_own], want[1][:n_own]) and int(want[1][:n_own].max()) > 0

    def canon(nm, num):
        cols = torch.arange(nm.shape[1], device=dev)[None, :] < num[:n_own, None]
        return torch.where(cols, nm[:n_own], torch.full_like(nm[:n_own], n)).sort(dim=1).values

    assert torch.equal(canon(got[0], got[1]), canon(want[0], want[1]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,n", [(torch.float64, 4097), (torch.float64, 1), (torch.float32, 4099)])
def test_peer_allreduce_kernel_sums_in_rank_order(dtype, n):
    """``p2p_allreduce`` over three buffers behind an address table (one device): scaled sum, vector body and scalar
    tail, float32 and float64; the float64 result equals the rank-ordered sum bit for bit."""
    dev = "cuda"
    g = torch.Generator().manual_seed(n)
    bufs = [torch.randn(n + 3, generator=g, dtype=dtype).to(dev)[:n] for _ in range(3)]
    bufs = [b.clone() for b in bufs]  # fresh allocations: 16-byte aligned starts
    ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    out = torch.empty(n, dtype=dtype, device=dev)
    torch.ops.nvalchemi.p2p_allreduce(ptrs, 3, 0.5, out)
    want = ((bufs[0] + bufs[1]) + bufs[2]) * 0.5
    assert torch.equal(out, want)
    with pytest.raises(RuntimeError, match="float32 or float64"):
        torch.ops.nvalchemi.p2p_allreduce(ptrs, 3, 1.0, torch.empty(8, dtype=torch.float16, device=dev))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float64, torch.float32])
def test_single_launch_push_allreduce_with_an_emulated_peer(dtype):
    """``p2p_allreduce_push`` on one device: the second "rank" is a plain buffer whose contribution and flags the test
    writes in advance (what that rank's kernel would have stored), so the kernel finds its peer already arrived.  Checks
    the sum, the values pushed into the peer's slots, the alternation of the two slot sets and several blocks."""
    from nvalchemi_toolkit_b200.parallel.symmetric import P2PContext, PeerReducer

    dev = torch.device("cuda", 0)
    small = PeerReducer.SMALL_BYTES
    ctx = P2PContext.single_process((1 << 20) + 4 * small + (1 << 16), dev, world=2)
    red = PeerReducer(None, dev, capacity_bytes=1 << 20, _context=ctx)
    esize = torch.empty(0, dtype=dtype).element_size()
    slot = small // esize
    mine_region = red.push_scratch.view(dtype).reshape(2, 2, slot)                 # [parity][rank][slot]
    off = ctx.arena.offset_of(red.push_scratch)
    peer_region = ctx.arena._bufs[1][off: off + 4 * small].view(dtype).reshape(2, 2, slot)
    flags = red.push_flags.view(16, 32)
    g = torch.Generator().manual_seed(3)
    for call, n in enumerate([20000, 1, 4097], start=1):
        x = torch.randn(n, generator=g, dtype=dtype).to(dev)
        peer = torch.randn(n, generator=g, dtype=dtype).to(dev)
        parity = call & 1
        mine_region[parity, 1, :n] = peer          # the peer's push into my slot set ...
        flags[:, 1] = call                          # ... and its flags, one per block
        x0, want = x.clone(), x + peer
        got = red(x)
        assert got is x and torch.equal(x, want)
        assert torch.equal(peer_region[parity, 0, :n], x0)  # my values arrived in the peer's slot for rank 0
        assert int(ctx.arena._bufs[1][ctx.arena.offset_of(red.push_flags):].view(torch.int32)[0]) == call
    assert red.small_calls == 3 and red.fallbacks == 0 and ctx.status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(8))
def test_native_neighbor_search_equals_brute_force_on_random_cells(seed):
    """Cell-list kernels on random triclinic cells with mixed periodicity, several systems per batch and both precisions
    against an explicit enumeration of periodic images (pairs within 1e-4 of the cutoff may fall on either side)."""
    import itertools
    import math

    from nvalchemi_toolkit_b200 import neighbors as nb

    g = torch.Generator().manual_seed(seed)
    dtype = torch.float64 if seed % 2 else torch.float32
    n_sys = 1 + seed % 3
    cutoff = 2.0 + 0.4 * seed
    cells, pbcs, poss, sizes = [], [], [], []
    for s in range(n_sys):
        cell = torch.diag(5.0 + 4.0 * torch.rand(3, generator=g, dtype=torch.float64))
        skew = 0.4 * torch.rand(1, generator=g).item()
        cell[1, 0], cell[2, 0], cell[2, 1] = skew * cell[0, 0], -skew * cell[0, 0], skew * cell[1, 1]
        n = int(torch.randint(20, 120, (1,), generator=g))
        cells.append(cell)
        pbcs.append(torch.rand(3, generator=g) < 0.7)
        poss.append((torch.rand(n, 3, generator=g, dtype=torch.float64) * 1.4 - 0.2) @ cell)  # some atoms outside the cell
        sizes.append(n)
    pos = torch.cat(poss)
    ptr = [0] + list(itertools.accumulate(sizes))
    bidx = torch.cat([torch.full((n,), s, dtype=torch.int32) for s, n in enumerate(sizes)])
    dev = "cuda"
    nm, num, sh = nb.neighbor_matrix(pos.to(dtype).to(dev), torch.stack(cells).to(dtype).to(dev), torch.stack(pbcs).to(dev),
                                     bidx.to(dev), torch.tensor(ptr, dtype=torch.int32, device=dev), cutoff, 1024)
    nm, num, sh = nm.cpu(), num.cpu(), sh.cpu()
    got = set()
    for i in range(pos.shape[0]):
        for k in range(int(num[i])):
            got.add((i, int(nm[i, k])) + tuple(int(x) for x in sh[i, k]))
    assert len(got) == int(num.sum())
    want, tol = set(), 1e-4
    borderline = set()
    for s in range(n_sys):
        cell, pbc, lo = cells[s], pbcs[s].tolist(), ptr[s]
        p = poss[s].to(dtype).double()  # the coordinates the kernel saw
        heights = 1.0 / torch.linalg.inv(cell).norm(dim=0)
        extent = (p @ torch.linalg.inv(cell))
        span = (extent.max(0).values - extent.min(0).values)
        reach = [int(math.ceil(cutoff / float(h) + float(w))) if per else 0 for h, w, per in zip(heights, span, pbc)]
        for shift in itertools.product(*[range(-r, r + 1) for r in reach]):
            d = (p[None, :, :] + torch.tensor(shift, dtype=torch.float64) @ cell - p[:, None, :]).norm(dim=-1)
            if shift == (0, 0, 0):
                d.fill_diagonal_(float("inf"))
            for i, j in (d < cutoff + tol).nonzero().tolist():
                entry = (lo + i, lo + j) + shift
                (want if d[i, j] < cutoff - tol else borderline).add(entry)
    assert want <= got and got <= (want | borderline), (len(want - got), len(got - want - borderline))
