# SPDX-License-Identifier: Apache-2.0
"""The six masked put / defrag operators (reference names, counters on the device) against plain PyTorch statements of the
same bookkeeping, on CPU and on the GPU."""
import pytest
import torch

from nvalchemi_toolkit_b200.ops import _native

pytestmark = pytest.mark.skipif(not _native.available(), reason="native library not built")
ops = torch.ops.nvalchemi


def _ref_put_per_system(src, smask, dst, dmask):
    dst, dmask = dst.clone(), dmask.clone()
    copied = torch.zeros_like(smask)
    empty = [i for i in range(dmask.numel()) if not dmask[i]]
    for i in range(smask.numel()):
        if smask[i] and empty:
            d = empty.pop(0)
            dst[d] = src[i]
            dmask[d] = True
            copied[i] = True
    return dst, dmask, copied


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.int64, torch.bool])
def test_put_and_defrag_per_system(device, dtype):
    g = torch.Generator().manual_seed(0)
    for n_src, n_dst in ((7, 5), (40, 64), (3000, 2100)):
        src = (torch.rand(n_src, 3, 3, generator=g) * 100).to(dtype)
        dst = torch.zeros(n_dst, 3, 3, dtype=dtype)
        smask = torch.rand(n_src, generator=g) < 0.6
        dmask = torch.rand(n_dst, generator=g) < 0.5
        want_dst, want_dmask, want_copied = _ref_put_per_system(src, smask, dst, dmask)
        s, sm, d, dm = (t.to(device) for t in (src, smask, dst, dmask))
        fit = torch.zeros(n_src, dtype=torch.bool, device=device)
        ops.compute_put_fit_mask_per_system(sm, dm, fit)
        assert torch.equal(fit.cpu(), want_copied) and torch.equal(dm.cpu(), dmask)  # the fit mask changes nothing
        copied = torch.zeros(n_src, dtype=torch.bool, device=device)
        ops.put_masked_per_system(s, sm, d, dm, copied)
        assert torch.equal(d.cpu(), want_dst) and torch.equal(dm.cpu(), want_dmask) and torch.equal(copied.cpu(), want_copied)
        # defrag: drop the copied rows of the source
        keep = ~want_copied
        want = torch.zeros_like(src)
        want[: int(keep.sum())] = src[keep]
        ops.defrag_per_system(s, copied)
        assert torch.equal(s.cpu(), want) and not bool(copied.any())


def _segments(g, n_seg, max_len):
    lens = torch.randint(0, max_len + 1, (n_seg,), generator=g)
    ptr = torch.zeros(n_seg + 1, dtype=torch.int32)
    ptr[1:] = torch.cumsum(lens, 0)
    return ptr


def test_put_and_defrag_segmented(device):
    g = torch.Generator().manual_seed(1)
    for n_seg, max_len, cap_rows, cap_seg, n_dst0 in ((6, 5, 18, 8, 2), (50, 30, 500, 40, 5), (1500, 9, 5000, 1800, 300)):
        sptr = _segments(g, n_seg, max_len)
        src = torch.randn(int(sptr[-1]), 4, generator=g)
        smask = torch.rand(n_seg, generator=g) < 0.5
        dptr = torch.zeros(cap_seg + 1, dtype=torch.int32)
        d0 = _segments(g, n_dst0, 3)
        dptr[: n_dst0 + 1] = d0
        dst = torch.zeros(cap_rows, 4)
        dst[: int(d0[-1])] = torch.randn(int(d0[-1]), 4, generator=g)
        # plain statement: segments in order, dropped when they do not fit; survivors packed without holes
        want_dst, want_ptr, nd, end = dst.clone(), dptr.clone(), n_dst0, int(d0[-1])
        cand = [i for i in range(n_seg) if smask[i]]
        for _ in range(2):
            off, rank, nxt = 0, 0, []
            for i in cand:
                ln = int(sptr[i + 1] - sptr[i])
                if end + off + ln <= cap_rows and n_dst0 + rank < cap_seg:
                    nxt.append(i)
                off, rank = off + ln, rank + 1
            cand = nxt
        want_copied = torch.zeros(n_seg, dtype=torch.bool)
        for i in cand:
            ln = int(sptr[i + 1] - sptr[i])
            want_dst[end: end + ln] = src[int(sptr[i]): int(sptr[i + 1])]
            end += ln
            nd += 1
            want_ptr[nd] = end
            want_copied[i] = True
        s, sp, sm, d, dp = (t.to(device) for t in (src, sptr, smask, dst, dptr))
        fit = torch.zeros(n_seg, dtype=torch.bool, device=device)
        ops.compute_put_fit_mask_segmented(sp, sm, dp, n_dst0, cap_rows, fit)
        assert torch.equal(fit.cpu(), want_copied)
        copied = torch.zeros(n_seg, dtype=torch.bool, device=device)
        count = torch.tensor([n_dst0], dtype=torch.int32, device=device)
        ops.put_masked_segmented(s, sp, sm, d, dp, copied, count, -1)  # count read from and written to the device
        assert int(count) == nd and torch.equal(copied.cpu(), want_copied)
        assert torch.equal(dp.cpu()[: nd + 1], want_ptr[: nd + 1]) and torch.equal(d.cpu(), want_dst)
        # defrag the source: drop what was copied
        keep = [i for i in range(n_seg) if not want_copied[i]]
        rows = torch.cat([src[int(sptr[i]): int(sptr[i + 1])] for i in keep]) if keep else src[:0]
        want_src = torch.zeros_like(src)
        want_src[: rows.shape[0]] = rows
        new_ptr = torch.zeros(n_seg + 1, dtype=torch.int32)
        lens = torch.tensor([int(sptr[i + 1] - sptr[i]) for i in keep], dtype=torch.int32)
        new_ptr[1: len(keep) + 1] = torch.cumsum(lens, 0)
        new_ptr[len(keep) + 1:] = rows.shape[0]
        kept = torch.zeros(1, dtype=torch.int32, device=device)
        ops.defrag_segmented(s, sp, copied, torch.empty_like(s), kept)
        assert int(kept) == len(keep) and torch.equal(sp.cpu(), new_ptr) and torch.equal(s.cpu(), want_src)
        assert not bool(copied.any())
