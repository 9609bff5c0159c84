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


def test_the_loader_reads_the_callers_row_order_on_the_host(tmp_path):
    """RowOrder::Shuffled with the permutations handed over by the caller: the rows every rank draws equal the
    checker's across epoch boundaries, over two files and two row ranges; needs no GPU (next_rows)."""
    width = SEQ + 1
    paths = [token_file(tmp_path, 13, 2, "a.bin")[0], token_file(tmp_path, 9, 0, "b.bin")[0]]
    spans = [(1, 8), (10, 21)]
    world, batch = 2, 2
    loaders = [ox.LitDataLoader.from_files(paths, batch, SEQ, rank=r, world_size=world, row_ranges=spans) for r in range(world)]
    n = loaders[0].num_rows()
    assert n == 18
    perm_of = lambda epoch: np.random.default_rng(77 + epoch).permutation(n).astype(np.uint32)  # noqa: E731
    ranges = hl.RowRanges(spans, 22)
    layout = hl.RowLayout(n, batch, world)
    for l in loaders:
        l.set_row_order(0, perm_of(0)).set_row_order(1, perm_of(1))
    pos = hl.DataPosition()
    for step in range(9):  # 4 global batches per epoch
        if step == 5:  # during epoch 1 the caller hands over epoch 2's order; epoch 0's is dropped
            for l in loaders:
                l.set_row_order(2, perm_of(2))
        for r, l in enumerate(loaders):
            want, _, _, nxt = hl.rank_window(layout, pos, r, SEQ, order=perm_of)
            assert l.next_rows() == [ranges.global_row(x) for x in want], (step, r)
        pos = nxt
    # epoch 3's order was never given: the batch that needs it says so
    for _ in range(3):
        loaders[0].next_rows()
    with pytest.raises(ox.OxzError, match="reads epoch 3 and the loader holds no row order for it"):
        loaders[0].next_rows()
    # not a permutation, or of another length: refused; None returns to stream order
    bad = perm_of(0).copy()
    bad[3] = bad[4]
    with pytest.raises(ox.OxzError, match="twice"):
        loaders[1].set_row_order(5, bad)
    with pytest.raises(ox.OxzError, match="holds 17 rows and the loader 18"):
        loaders[1].set_row_order(5, perm_of(0)[:17])
    loaders[1].set_row_order(0, None)
    loaders[1].seek(ox.DataPosition(0, 0))
    assert loaders[1].next_rows() == [ranges.global_row(x) for x in (2, 3)]
    with pytest.raises(ox.OxzError, match="mixture"):
        loaders[0].with_mixture([1.0, 1.0])
    for l in loaders:
        l.close()


@pytest.mark.gpu
@pytest.mark.parametrize("depth", [0, 2])
def test_shuffled_batches_carry_the_tokens_of_the_permuted_rows(tmp_path, depth):
    """The same on the device, with and without the prefetch thread: inputs and targets are the tokens of the rows the
    caller's permutation names, bit for bit, across two epoch boundaries."""
    import torch
    from oxidizr_b200.interop import device_view
    rows, batch, world = 14, 2, 2
    path, toks = token_file(tmp_path, rows, 3)
    perm_of = lambda epoch: np.random.default_rng(5 + epoch).permutation(rows).astype(np.uint32)  # noqa: E731
    loaders = [ox.LitDataLoader(path, batch, SEQ, rank=r, world_size=world) for r in range(world)]
    for l in loaders:
        l.set_row_order(0, perm_of(0)).set_row_order(1, perm_of(1))
        if depth:
            l.with_prefetch(depth)
    layout, pos = hl.RowLayout(rows, batch, world), hl.DataPosition()
    for step in range(8):  # 3 global batches per epoch
        if step == 4:
            for l in loaders:
                l.set_row_order(2, perm_of(2))
        for r, l in enumerate(loaders):
            i_ptr, t_ptr, got_rows = l.next_batch()
            torch.cuda.synchronize()
            inputs = device_view(i_ptr, batch * SEQ * 8, torch.int64).cpu().numpy().reshape(batch, SEQ)
            targets = device_view(t_ptr, batch * SEQ * 8, torch.int64).cpu().numpy().reshape(batch, SEQ)
            want_rows, want_in, want_tg, nxt = hl.rank_window(layout, pos, r, SEQ, order=perm_of)
            assert got_rows == want_rows, (step, r)
            assert np.array_equal(inputs, toks[np.array(want_in)].astype(np.int64))
            assert np.array_equal(targets, toks[np.array(want_tg)].astype(np.int64))
        pos = nxt
    for l in loaders:
        l.close()


def write_tokens(tmp_path, tokens, name):
    path = tmp_path / name
    np.asarray(tokens, dtype="<u4").tofile(path)
    return str(path)


def draw(loader, batch, seq):
    """One batch with its masks, read back: (inputs, targets, loss_mask|None, scored, offsets|None, ids|None)."""
    import torch
    from oxidizr_b200.interop import device_view
    i, t, _ = loader.next_batch()
    m = loader.batch_masks()
    torch.cuda.synchronize()
    n = batch * seq
    view = lambda addr, dt, count: device_view(addr, count * torch.empty(0, dtype=dt).element_size(), dt, 0).cpu().tolist()  # noqa: E731
    mask = view(m["loss_mask"], torch.float32, n) if m["loss_mask"] else None
    ids = view(m["segment_ids"], torch.int32, n) if m["segment_ids"] else None
    offsets = view(m["cu_seqlens"], torch.int32, m["n_segments"]() + 1) if m["cu_seqlens"] else None
    return view(i, torch.int64, n), view(t, torch.int64, n), mask, m["scored"](), offsets, ids


@pytest.mark.gpu
def test_masks_and_segments_give_the_reference_tests_answers(tmp_path):
    SEP, EOS, BASE = 0, 3, 12
    # src/data/host_masks.rs:115-124
    l = ox.LitDataLoader(write_tokens(tmp_path, [5, 6, SEP, 7, 8, 9], "a.bin"), 1, 5).with_document_mask(SEP)
    _, _, mask, scored, offsets, ids = draw(l, 1, 5)
    assert (mask, scored, offsets, ids) == ([1.0, 1.0, 0.0, 1.0, 1.0], 4, [0, 3, 5], [0, 0, 0, 1, 1])
    l.close()
    # src/data/host_masks.rs:126-137: the document mask ANDs with the target mask
    l = ox.LitDataLoader(write_tokens(tmp_path, [4, BASE, SEP, BASE + 1, 4], "b.bin"), 1, 4)
    _, _, mask, scored, _, _ = draw(l.with_target_mask(BASE, [EOS]).with_document_mask(SEP), 1, 4)
    assert (mask, scored) == ([1.0, 0.0, 0.0, 0.0], 1)
    l.close()
    # src/data/host_masks.rs:139-146: off leaves no mask and no segments, every position scores
    l = ox.LitDataLoader(write_tokens(tmp_path, [5, SEP, 6], "c.bin"), 1, 2)
    assert draw(l, 1, 2)[2:] == (None, 2, None, None)
    l.close()
    # src/data/segments.rs:144-169
    for tokens, b, s, want_off, want_ids in [
            ([5, 6, 7, 1, 8, SEP, 9, 2], 2, 3, [0, 3, 5, 6], [0, 0, 0, 1, 1, 2]),
            ([SEP, SEP, 5, 6], 1, 3, [0, 1, 2, 3], [0, 1, 2]),
            ([5, SEP, 3, 6, SEP, 4], 2, 2, [0, 2, 4], [0, 0, 1, 1]),
            ([5, 6, 7, 8, 9, 10], 2, 2, [0, 2, 4], [0, 0, 1, 1])]:
        l = ox.LitDataLoader(write_tokens(tmp_path, tokens, "d.bin"), b, s).with_document_mask(SEP)
        _, _, _, _, offsets, ids = draw(l, b, s)
        assert (offsets, ids) == (want_off, want_ids), tokens
        l.close()
    # src/data/mask.rs:222-274: prefix-LM scoring, the boundary, a row that starts mid-sequence
    l = ox.LitDataLoader(write_tokens(tmp_path, [0, 1, 4, 5, 6, 7, 2, 12, 13, 14, 15, 16, 17, 18, EOS], "e.bin"), 1, 14)
    assert draw(l.with_target_mask(BASE, [EOS]), 1, 14)[2] == [0.0] * 6 + [1.0] * 8
    l.close()
    l = ox.LitDataLoader(write_tokens(tmp_path, [0, BASE - 1, BASE, BASE + 1], "f.bin"), 1, 3).with_target_mask(BASE, [EOS])
    assert draw(l, 1, 3)[2] == [0.0, 1.0, 1.0]
    l.close()
    l = ox.LitDataLoader(write_tokens(tmp_path, [0, 1, 4, 2, 12, 13, EOS, 0, 1, 5, 6, 2, 13, 14, EOS], "g.bin"), 1, 4)
    l.with_target_mask(BASE, [EOS])
    assert draw(l, 1, 4)[2] == [0.0, 0.0, 0.0, 1.0] and draw(l, 1, 4)[2] == [1.0, 0.0, 0.0, 0.0]
    l.close()


@pytest.mark.gpu
@pytest.mark.parametrize("batch,seq,world,sep_every", [(2, 3, 2, 5), (3, 700, 1, 37), (5, 257, 2, 2), (4, 1024, 1, 100000), (300, 9, 1, 4)])
def test_masks_equal_the_checkers_on_every_rank_and_batch(tmp_path, batch, seq, world, sep_every):
    """Long rows (several 256-position chunks), many rows (several scan chunks), dense and absent separators: the loss
    mask, the scored count, the segment ids and offsets equal the checker's for every rank, and the ranks' offsets
    concatenate to the global batch's (src/data/host_masks.rs:170-198)."""
    SEP, BASE, ALWAYS = 7, 40, [3, 11]
    width = seq + 1
    rows = batch * world * 3 + 1
    rng = np.random.default_rng(batch * 1000 + seq)
    toks = rng.integers(8, 64, size=rows * width + 2, dtype=np.uint32)
    toks[rng.integers(0, toks.size, size=toks.size // sep_every)] = SEP
    toks[rng.integers(0, toks.size, size=toks.size // 9)] = 3
    path = write_tokens(tmp_path, toks, "t.bin")
    loaders = [ox.LitDataLoader(path, batch, seq, rank=r, world_size=world).with_target_mask(BASE, ALWAYS).with_document_mask(SEP)
               for r in range(world)]
    whole = hl.RowLayout(rows, batch * world)
    ranked = hl.RowLayout(rows, batch, world)
    pos = hl.DataPosition()
    for _ in range(4):  # crosses an epoch boundary
        g_rows, _, _, nxt = hl.rank_window(whole, pos, 0, seq)
        g_window = [int(t) for r in g_rows for t in toks[r * width:(r + 1) * width]]
        _, g_scored, (g_off, _) = hl.host_masks(g_window, batch * world, seq, (BASE, ALWAYS), SEP)
        joined, scored = [0], 0
        for r, l in enumerate(loaders):
            rr, _, _, _ = hl.rank_window(ranked, pos, r, seq)
            window = [int(t) for row in rr for t in toks[row * width:(row + 1) * width]]
            want_mask, want_scored, (want_off, want_ids) = hl.host_masks(window, batch, seq, (BASE, ALWAYS), SEP)
            inputs, targets, mask, got_scored, offsets, ids = draw(l, batch, seq)
            assert inputs == [window[b * width + s] for b in range(batch) for s in range(seq)]
            assert targets == [window[b * width + s + 1] for b in range(batch) for s in range(seq)]
            assert mask == want_mask and got_scored == want_scored
            assert offsets == want_off and ids == want_ids
            joined += [o + r * batch * seq for o in offsets[1:]]
            scored += got_scored
        assert joined == g_off and scored == g_scored
        pos = nxt
    for l in loaders:
        l.close()


def test_mask_settings_are_checked_on_the_host(tmp_path):
    path = write_tokens(tmp_path, list(range(40)), "h.bin")
    l = ox.LitDataLoader(path, 2, 3)
    with pytest.raises(ox.OxzError, match="at most 16"):
        l.with_target_mask(5, list(range(17)))
    with pytest.raises(ox.OxzError, match="no batch has been drawn"):
        l.batch_masks()
    l.close()


def test_several_files_and_row_ranges_are_checked_on_the_host(tmp_path):
    width = SEQ + 1
    a = write_tokens(tmp_path, list(range(6 * width + 1)), "s0.bin")
    b = write_tokens(tmp_path, list(range(4 * width + 3)), "s1.bin")
    c = write_tokens(tmp_path, [1, 2], "s2.bin")  # shorter than a row: no rows
    l = ox.LitDataLoader.from_files([a, b, c], 2, SEQ)
    assert l.source_rows() == [6, 4, 0] and l.num_rows() == 10
    l.close()
    l = ox.LitDataLoader.from_files([a, b], 2, SEQ, row_ranges=[(0, 5), (6, 9)])
    assert l.num_rows() == 8
    l.close()
    for ranges, msg in [([(3, 3)], "not a non-empty range"), ([(0, 11)], "inside the 10 whole rows"),
                        ([(0, 5), (4, 6)], "starts before row 5")]:
        with pytest.raises(ox.OxzError, match=msg):
            ox.LitDataLoader.from_files([a, b], 1, SEQ, row_ranges=ranges)
    with pytest.raises(ox.OxzError, match="no data files given"):
        ox.LitDataLoader.from_files([], 1, SEQ)
    with pytest.raises(ox.OxzError, match="failed to open data file"):
        ox.LitDataLoader.from_files([a, str(tmp_path / "gone.bin")], 1, SEQ)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [1, 2])
def test_batches_over_several_files_and_ranges_read_the_checkers_rows(tmp_path, world):
    """src/data/multi_source.rs:99-161 in stream order: rows follow the sources in order, no row crosses a file seam or
    touches a tail, train and eval ranges stay disjoint, a batch can carry rows of several sources."""
    width = SEQ + 1
    lens = [6 * width + 1, 4 * width + 3, 2, 5 * width]
    rng = np.random.default_rng(5)
    sources = [rng.integers(0, 50000, size=n, dtype=np.uint32) for n in lens]
    paths = [write_tokens(tmp_path, t, f"m{i}.bin") for i, t in enumerate(sources)]
    total = sum(n // width for n in lens)
    train_spans, eval_spans = [(0, 5), (6, 9), (10, 15)], [(5, 6), (9, 10)]
    batch = 2
    for spans in (train_spans, eval_spans, None):
        ranges = hl.RowRanges(spans or [(0, total)], total)
        if ranges.len < batch * world:
            continue
        layout = hl.RowLayout(ranges.len, batch, world)
        loaders = [ox.LitDataLoader.from_files(paths, batch, SEQ, rank=r, world_size=world, row_ranges=spans) for r in range(world)]
        pos = hl.DataPosition()
        seen = []
        for _ in range(2 * layout.batches_per_epoch() + 1):
            for r, l in enumerate(loaders):
                loader_rows, _, _, nxt = hl.rank_window(layout, pos, r, SEQ)
                want_rows = [ranges.global_row(x) for x in loader_rows]
                window = [t for g in want_rows for t in hl.store_row(sources, width, g)]
                i, t, rows = l.next_batch()
                inputs, targets = read_i64(i, batch * SEQ), read_i64(t, batch * SEQ)
                assert rows == want_rows
                assert inputs == [int(window[b * width + s]) for b in range(batch) for s in range(SEQ)]
                assert targets == [int(window[b * width + s + 1]) for b in range(batch) for s in range(SEQ)]
                seen += rows
            pos = nxt
        allowed = {g for a, b in (spans or [(0, total)]) for g in range(a, b)}
        assert set(seen) <= allowed
        for l in loaders:
            l.close()


def read_i64(addr, count):
    import torch
    from oxidizr_b200.interop import device_view
    torch.cuda.synchronize()
    return device_view(addr, count * 8, torch.int64, 0).cpu().tolist()


# ---- weighted mixtures in stream order (host only: the row order needs no GPU)
def mixed(tmp_path, rows, batch, **kw):
    """Sources of rows[i] rows whose tokens are their own offsets in the concatenation (src/data/mixture/loader.rs:94-106)."""
    width = SEQ + 1
    first, paths = 0, []
    for i, n in enumerate(rows):
        paths.append(write_tokens(tmp_path, list(range(first, first + n * width)), f"mix{i}.bin"))
        first += n * width
    return ox.LitDataLoader.from_files(paths, batch, SEQ, **kw)


def epoch_rows(loader, batches):
    return [r for _ in range(batches) for r in loader.next_rows()]


def test_mixture_quotas_follow_the_reference_cases():
    # src/data/mixture/quota.rs:63-90
    assert ox.mixture_quotas([3.0, 1.0], 100) == [75, 25] and ox.mixture_quotas([1.0, 1.0, 2.0], 8) == [2, 2, 4]
    assert ox.mixture_quotas([1.0, 1.0, 1.0], 10) == [4, 3, 3] and ox.mixture_quotas([1.0, 1.0, 1.0], 11) == [4, 4, 3]
    assert ox.mixture_quotas([1.0, 2.0, 3.0, 4.0], 12) == [1, 2, 4, 5] and ox.mixture_quotas([2.0, 2.0], 1) == [1, 0]
    assert ox.mixture_quotas([0.25], 37) == [37]
    rng = np.random.default_rng(3)
    for _ in range(200):
        w = [float(x) for x in rng.uniform(1e-3, 5.0, size=int(rng.integers(1, 7)))]
        rows = int(rng.integers(1, 20000))
        assert ox.mixture_quotas(w, rows) == hl.mixture_quotas(w, rows)
    for bad in (0.0, -1.0, float("nan"), float("inf")):
        with pytest.raises(ox.OxzError, match=r"trainer.data.sources\[2\].weight"):
            ox.mixture_quotas([1.0, 1.0, bad], 10)


def test_the_layout_counts_rows_per_epoch(tmp_path):
    # src/data/mixture/loader.rs:108-122
    l = mixed(tmp_path, [10, 4], 2).with_mixture([1.0, 1.0], 20)
    assert l.num_rows() == 20
    sources = l.mixture_sources()
    assert sources[1]["rows_per_epoch"] == 10 and sources[1]["repeats"] == 2.5 and sources[1]["train_rows"] == 4
    l.close()
    plain = mixed(tmp_path, [3], 1)
    assert plain.mixture_sources() is None
    plain.close()


def test_a_mixture_reads_only_the_row_ranges_and_fills_its_quotas(tmp_path):
    # src/data/mixture/loader.rs:124-141: sources [0,8) and [8,14); train [0,6) and [8,12); quotas 3 and 7 of 10
    l = mixed(tmp_path, [8, 6], 2, row_ranges=[(0, 6), (8, 12)]).with_mixture([1.0, 2.0])
    assert l.num_rows() == 10
    rows = epoch_rows(l, 15)
    assert all(r < 6 or 8 <= r < 12 for r in rows)
    assert sum(r < 6 for r in rows) == 9
    l.close()


def test_one_weighted_source_reads_what_the_plain_loader_reads(tmp_path):
    # src/data/mixture/loader.rs:143-152, src/data/mixture/state.rs:268-283
    plain, weighted = mixed(tmp_path, [12], 3), mixed(tmp_path, [12], 3).with_mixture([5.0])
    assert epoch_rows(weighted, 16) == epoch_rows(plain, 16)
    for l in (plain, weighted):
        l.close()


def test_an_upsampled_source_repeats_every_row_once_per_pass(tmp_path):
    # src/data/mixture/state.rs:231-246 and draw.rs:130-137 in stream order
    l = mixed(tmp_path, [3, 8], 1, row_ranges=[(0, 3), (3, 11)]).with_mixture([1.0, 1.0], 16)
    rows = epoch_rows(l, 48)
    small = [r for r in rows if r < 3]
    assert len(small) == 24 and all(sorted(small[i:i + 3]) == [0, 1, 2] for i in range(0, 24, 3))
    assert small[:7] == [0, 1, 2, 0, 1, 2, 0]
    l.close()


def test_a_seek_mid_epoch_continues_the_uninterrupted_rows(tmp_path):
    # src/data/mixture/loader.rs:154-171
    make = lambda: mixed(tmp_path, [9, 2], 3).with_mixture([1.0, 1.0], 12)  # noqa: E731
    full = make()
    epoch_rows(full, 5)
    resumed = make()
    resumed.seek(hl_advance(12, 3, 5))
    assert epoch_rows(resumed, 9) == epoch_rows(full, 9)
    for l in (full, resumed):
        l.close()


def hl_advance(num_rows, batch, batches):
    p = hl.RowLayout(num_rows, batch).advance(hl.DataPosition(), batches)
    return ox.DataPosition(p.epoch, p.row)


@pytest.mark.parametrize("world", [1, 2])
def test_mixture_rows_equal_the_checkers_for_every_rank(tmp_path, world):
    rows, spans, weights, per_epoch, batch = [700, 3, 190, 40], [(0, 650), (700, 703), (710, 880)], [2.0, 1.0, 1.0], 9000, 5
    loaders = [mixed(tmp_path, rows[:3], batch, rank=r, world_size=world, row_ranges=spans).with_mixture(weights, per_epoch)
               for r in range(world)]
    total = sum(rows[:3])
    mix = hl.Mixture(weights, per_epoch, hl.source_train_rows(rows[:3], spans, total))
    layout = hl.RowLayout(per_epoch, batch, world)
    pos = hl.DataPosition()
    # jump to the end of the first epoch, then cross into the second
    skip = layout.batches_per_epoch() - 3
    pos = layout.advance(pos, skip)
    for l in loaders:
        l.seek(ox.DataPosition(pos.epoch, pos.row))
    for _ in range(8):
        start = layout.batch_start(pos)
        for r, l in enumerate(loaders):
            slots = [start.row + r * batch + k for k in range(batch)]
            assert l.next_rows() == [mix.global_row(start.epoch, s) for s in slots]
        pos = hl.DataPosition(start.epoch, start.row + layout.batch_size())
    for l in loaders:
        l.close()


def test_bad_mixtures_are_refused_naming_the_key(tmp_path):
    # src/data/mixture/state.rs:285-316, 217-229
    for weights, per_epoch, msg in [([1.0], None, r"1 weight\(s\), and the loader reads 2 source\(s\)"),
                                    ([1.0, -2.0], None, r"trainer.data.sources\[1\].weight is -2"),
                                    ([1.0, 1.0], 0, "trainer.data.rows_per_epoch is 0"),
                                    ([1.0, 1.0], (1 << 28) + 1, str(1 << 28))]:
        l = mixed(tmp_path, [4, 4], 1)
        with pytest.raises(ox.OxzError, match=msg):
            l.with_mixture(weights, per_epoch)
        l.close()
    l = mixed(tmp_path, [4, 4], 1, row_ranges=[(0, 4)])
    with pytest.raises(ox.OxzError, match=r"trainer.data.sources\[1\] holds no training rows"):
        l.with_mixture([1.0, 1.0])
    l.close()


@pytest.mark.gpu
def test_mixture_batches_carry_the_tokens_of_the_rows_they_name(tmp_path):
    """Every token of the mixed sources is its own offset in the concatenation, so a batch's inputs must be
    row * width + s for the rows the loader names (src/data/positioning.rs tests' rows_of)."""
    width = SEQ + 1
    l = mixed(tmp_path, [9, 2, 5], 3, row_ranges=[(0, 8), (9, 16)]).with_mixture([1.0, 1.0, 2.0], 24)
    twin = mixed(tmp_path, [9, 2, 5], 3, row_ranges=[(0, 8), (9, 16)]).with_mixture([1.0, 1.0, 2.0], 24)
    for _ in range(20):
        i, t, rows = l.next_batch()
        assert rows == twin.next_rows()
        assert read_i64(i, 3 * SEQ) == [r * width + s for r in rows for s in range(SEQ)]
        assert read_i64(t, 3 * SEQ) == [r * width + s + 1 for r in rows for s in range(SEQ)]
    l.close()
    twin.close()


@pytest.mark.gpu
@pytest.mark.parametrize("depth", [1, 3])
def test_the_prefetch_loader_yields_the_sync_loaders_batches(tmp_path, depth):
    """src/data/prefetch.rs:350-390 and src/data/host_masks.rs:148-168: over several epochs, after a seek, with the
    masks on and under a mixture, a loader with a prefetch thread hands out exactly the batches of one without."""
    SEP = 0
    width = SEQ + 1
    rng = np.random.default_rng(11)
    lens = [40 * width + 2, 23 * width]
    paths = []
    for i, n in enumerate(lens):
        toks = rng.integers(1, 9, size=n, dtype=np.uint32)
        toks[rng.integers(0, n, size=n // 7)] = SEP
        paths.append(write_tokens(tmp_path, toks, f"p{i}.bin"))
    make = lambda: (ox.LitDataLoader.from_files(paths, 2, SEQ, rank=1, world_size=2, row_ranges=[(0, 35), (40, 60)])  # noqa: E731
                    .with_mixture([1.0, 2.0], 30).with_target_mask(4, [2]).with_document_mask(SEP))
    sync, pre = make(), make().with_prefetch(depth)
    start = hl_advance(30, 4, 3)
    for l in (sync, pre):
        l.seek(start)
    with pytest.raises(ox.OxzError, match="prefetch thread draws"):
        pre.next_rows()
    for n in range(25):  # more than three epochs of 7 batches
        a, b = draw_with_rows(sync, 2, SEQ), draw_with_rows(pre, 2, SEQ)
        assert a == b, f"batch {n}"
        assert sync.position() == pre.position()
    # a seek in the middle restarts the thread at the new position
    back = hl_advance(30, 4, 9)
    for l in (sync, pre):
        l.seek(back)
    for n in range(5):
        assert draw_with_rows(sync, 2, SEQ) == draw_with_rows(pre, 2, SEQ)
    pre.with_prefetch(0)  # off again: the loader goes on from where it stands
    assert draw_with_rows(sync, 2, SEQ) == draw_with_rows(pre, 2, SEQ)
    for l in (sync, pre):
        l.close()


def draw_with_rows(loader, batch, seq):
    import torch
    from oxidizr_b200.interop import device_view
    i, t, rows = loader.next_batch()
    m = loader.batch_masks()
    torch.cuda.synchronize()
    n = batch * seq
    view = lambda addr, dt, count: device_view(addr, count * torch.empty(0, dtype=dt).element_size(), dt, 0).cpu().tolist()  # noqa: E731
    return (rows, view(i, torch.int64, n), view(t, torch.int64, n), view(m["loss_mask"], torch.float32, n), m["scored"](),
            view(m["segment_ids"], torch.int32, n), view(m["cu_seqlens"], torch.int32, m["n_segments"]() + 1))
