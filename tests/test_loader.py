"""The rank-sliced stream-order loader: token indices bit-exact against the checker's row arithmetic
(src/data/ranks.rs:54-185, src/data/positioning.rs:72-200, tests/data_ranks.rs:94-122)."""
import numpy as np
import pytest

import oxidizr_b200 as ox
from oracle import host_logic as hl

SEQ = 3
WIDTH = SEQ + 1


def token_file(tmp_path, rows, tail, name="tokens.bin"):
    toks = ((np.arange(rows * WIDTH + tail, dtype=np.uint64) * 2654435761) % 100003).astype("<u4")
    path = tmp_path / name
    toks.tofile(path)
    return str(path), toks


def test_open_counts_whole_rows_and_refuses_bad_ranges(tmp_path):
    path, _ = token_file(tmp_path, 23, 2)
    l = ox.LitDataLoader(path, 3, SEQ, rank=1, world_size=2)
    assert l.num_rows() == 23 and l.position() == ox.DataPosition(0, 0)
    l.close()
    l = ox.LitDataLoader(path, 2, SEQ, first_row=3, end_row=17)
    assert l.num_rows() == 14
    with pytest.raises(ox.OxzError, match="past this shard's 14 rows"):
        l.seek(ox.DataPosition(0, 15))
    l.close()
    for kw, msg in [(dict(rank=2, world_size=2), "rank 2 is not below world size 2"),
                    (dict(world_size=0), "world size is 0"),
                    (dict(first_row=4, end_row=4), "does not fit the data's 23 whole rows"),
                    (dict(end_row=24), "does not fit the data's 23 whole rows")]:
        with pytest.raises(ox.OxzError, match=msg):
            ox.LitDataLoader(path, 3, SEQ, **kw)
    with pytest.raises(ox.OxzError, match="one global batch of 24 rows"):
        ox.LitDataLoader(path, 3, SEQ, world_size=8)
    odd = tmp_path / "odd.bin"
    odd.write_bytes(b"\x00" * 10)
    with pytest.raises(ox.OxzError, match="not a multiple of 4"):
        ox.LitDataLoader(str(odd), 1, SEQ)
    with pytest.raises(ox.OxzError, match="failed to open data file"):
        ox.LitDataLoader(str(tmp_path / "absent.bin"), 1, SEQ)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,batch,world,first,end", [(23, 3, 2, 0, 0), (11, 1, 3, 0, 0), (20, 2, 2, 3, 17), (10, 3, 1, 0, 0)])
def test_rank_batches_hold_exactly_the_checkers_token_indices(tmp_path, rows, batch, world, first, end):
    import torch
    from oxidizr_b200.interop import device_view
    path, toks = token_file(tmp_path, rows, 1)
    loaders = [ox.LitDataLoader(path, batch, SEQ, rank=r, world_size=world, first_row=first, end_row=end) for r in range(world)]
    layout = hl.RowLayout((end or rows) - first, batch, world)
    pos = hl.DataPosition()
    for step in range(12):
        nxt = None
        union = []
        for r, l in enumerate(loaders):
            i_ptr, t_ptr, got_rows = l.next_batch()
            torch.cuda.synchronize()
            inputs = device_view(i_ptr, batch * SEQ * 8, torch.int64).cpu().numpy().reshape(batch, SEQ)
            targets = device_view(t_ptr, batch * SEQ * 8, torch.int64).cpu().numpy().reshape(batch, SEQ)
            want_rows, want_in, want_tg, nxt = hl.rank_window(layout, pos, r, SEQ, first)
            assert got_rows == want_rows, (step, r)
            assert inputs.dtype == np.int64 and np.array_equal(inputs, toks[np.array(want_in)].astype(np.int64))
            assert np.array_equal(targets, toks[np.array(want_tg)].astype(np.int64))
            assert (l.position().epoch, l.position().row) == (nxt.epoch, nxt.row)
            union += got_rows
        # the ranks' windows concatenate to the global window, each row once
        assert len(set(union)) == batch * world and union == list(range(union[0], union[0] + batch * world))
        pos = nxt
    # resume: a fresh loader seeks a saved position and continues with the same rows (tests/exact_resume.rs)
    saved = loaders[0].position()
    a = loaders[0].next_batch()[2]
    fresh = ox.LitDataLoader(path, batch, SEQ, rank=0, world_size=world, first_row=first, end_row=end)
    fresh.seek(saved)
    assert fresh.next_batch()[2] == a
    for l in loaders + [fresh]:
        l.close()
