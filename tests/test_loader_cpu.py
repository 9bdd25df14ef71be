"""The sharded token loader (gptb200_loader_*) against the reference's own DataLoader (src/train/data_loader.cpp, compiled
unmodified into oracle/_ref): with one rank the batches are identical, epoch after epoch, for the same srand seed; with several
ranks the ranks' shards put side by side are the batch a single process with the global batch size would see.  No GPU."""
import numpy as np
import pytest

SEQ = 16


@pytest.fixture(scope="module")
def token_file(tmp_path_factory):
    rng = np.random.default_rng(7)
    path = tmp_path_factory.mktemp("tokens") / "train.bin"
    rng.integers(0, 50257, size=SEQ * 41 + 5).astype(np.uint16).tofile(path)   # 40 samples per epoch, ragged tail
    return str(path)


def _ours(token_file, seed, epochs, world, batch, max_batches):
    import gpt_b200
    loaders = [gpt_b200.Loader(token_file, SEQ) for _ in range(world)]
    out = []
    for r, ld in enumerate(loaders):   # every rank draws the same random numbers: seed before each rank's run
        gpt_b200.Loader.seed_libc_rand(seed)
        batches = []
        for _ in range(epochs):
            ld.reset_epoch()
            for _ in range(max_batches):
                b = ld.next_batch(r, world, batch)
                if b is None:
                    break
                batches.append(b)
        out.append(batches)
        ld.close()
    return out


def test_one_rank_reproduces_the_reference_loader(built_library, reference, token_file):
    ref_in, ref_lbl = reference.loader_batches(token_file, 4, SEQ, 42, 3, 100)
    ours = _ours(token_file, 42, 3, 1, 4, 100)[0]
    assert len(ours) == len(ref_in) == 3 * 10
    for (i, l), ri, rl in zip(ours, ref_in, ref_lbl):
        assert np.array_equal(i, ri) and np.array_equal(l, rl)
    assert np.array_equal(ref_in[0][:, 1:], ref_lbl[0][:, :-1])     # labels are the inputs shifted by one token


@pytest.mark.parametrize("world", [2, 4])
def test_shards_put_together_are_the_global_batch(built_library, reference, token_file, world):
    per_rank = 2
    ref_in, ref_lbl = reference.loader_batches(token_file, world * per_rank, SEQ, 9, 2, 100)
    ours = _ours(token_file, 9, 2, world, per_rank, 100)
    assert all(len(b) == len(ref_in) for b in ours)
    for step in range(len(ref_in)):
        got_in = np.concatenate([ours[r][step][0] for r in range(world)])
        got_lbl = np.concatenate([ours[r][step][1] for r in range(world)])
        assert np.array_equal(got_in, ref_in[step]) and np.array_equal(got_lbl, ref_lbl[step])


def test_bad_files_and_arguments(built_library, tmp_path):
    import gpt_b200
    with pytest.raises(gpt_b200.GptB200Error):
        gpt_b200.Loader(str(tmp_path / "missing.bin"), SEQ)
    short = tmp_path / "short.bin"
    np.zeros(2 * SEQ, np.uint16).tofile(short)       # not even one batch (data_loader.cpp:95-100)
    with pytest.raises(gpt_b200.GptB200Error):
        gpt_b200.Loader(str(short), SEQ)
    ok = tmp_path / "ok.bin"
    np.arange(SEQ * 8, dtype=np.uint16).tofile(ok)
    ld = gpt_b200.Loader(str(ok), SEQ)
    assert ld.num_samples == 7
    ld.reset_epoch()
    with pytest.raises(gpt_b200.GptB200Error):
        ld.next_batch(2, 2, 1)                        # rank outside the world
    assert ld.next_batch(0, 1, 8) is None             # more than the epoch holds
    ld.close()
