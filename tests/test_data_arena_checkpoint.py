"""Tokenizer / batcher semantics (FINAL_CLEAN_CODE_/src/data/dataset.cpp:19-79), flat arena order
(FINAL_CLEAN_CODE_/src/model/transformer.cu:171-188), bucket coalescing (:428-457), checkpoint round trip
and the trajectory hash (FINAL_CLEAN_CODE_/src/main.cu:40-65)."""
import numpy as np
import pytest
import torch

from cme213_final_project_b200 import checkpoint as ckpt
from cme213_final_project_b200.arena import ArenaLayout, init_flat, xorshift_uniform
from cme213_final_project_b200.config import ModelConfig, preset
from cme213_final_project_b200.data import CharTokenizer, Dataset, ShardPlan, synthetic_batches, synthetic_tokens


def test_tokenizer_sorted_vocab_and_unknown_skip():
    tok = CharTokenizer().build(b"hello world")
    assert tok.vocab_size == 8 and bytes(tok.id_to_char) == b" dehlorw"
    ids = tok.encode(b"hold!z")
    assert tok.decode(ids) == b"hold"


def test_batcher_chunks_and_cursor():
    tokens = np.arange(100, dtype=np.int32)
    ds = Dataset(tokens, seq_len=4, batch_size=3)
    assert ds.num_batches() == (100 - 1) // 15 == 6
    x, y = ds.next_batch()
    assert x.tolist() == [0, 1, 2, 3, 5, 6, 7, 8, 10, 11, 12, 13]
    assert y.tolist() == [1, 2, 3, 4, 6, 7, 8, 9, 11, 12, 13, 14]
    x2, _ = ds.next_batch()
    assert x2[0] == 15
    ax, ay = ds.all_batches()
    assert ax.shape == (6, 12) and ax[1].tolist() == x2.tolist() and ax.dtype == torch.int32
    ds.reset()
    n = 0
    while ds.next_batch() is not None:
        n += 1
    assert n == 6


def test_reference_corpus_counts():
    import os
    from cme213_final_project_b200.data import reference_corpus_path
    path = reference_corpus_path()
    if not os.path.exists(path):
        pytest.skip("corpus not present")
    from cme213_final_project_b200.data import read_file
    text = read_file(path)
    tok = CharTokenizer().build(text)
    ds = Dataset(tok.encode(text), 64, 32)
    assert tok.vocab_size == 65 and len(ds.tokens) == 1115394 and ds.num_batches() == 536


def test_shard_plan_drops_remainder():
    p = ShardPlan(536, 3)
    assert p.local_batches == 178 and p.dropped == 2 and p.batch_index(5, 2) == 17


def test_synthetic_is_seeded_and_in_range():
    a, b = synthetic_tokens(65, 1000, 0), synthetic_tokens(65, 1000, 0)
    assert (a == b).all() and a.min() >= 0 and a.max() < 65
    x, y = synthetic_batches(65, 64, 8, 5, seed=0)
    assert x.shape == (5, 512) and (x[0, 1:64] == y[0, 0:63]).all()


def test_arena_order_is_the_reference_order():
    m, _ = preset("parity-h128")
    L = ArenaLayout(m)
    assert [s.name for s in L.specs] == ["Wout", "W2", "b2", "W1", "b1", "ln2_gamma", "ln2_beta", "Wo", "Wq", "Wk",
                                         "Wv", "ln1_gamma", "ln1_beta", "tok_embed", "pos_embed"]
    assert L.num_params() == 222592 == L.total
    assert ArenaLayout(preset("parity-h256")[0]).num_params() == 838400
    assert ArenaLayout(preset("parity-h512")[0]).num_params() == 3249664
    sizes = [b.numel for b in L.natural_buckets]
    D, FF, V, T = 128, 512, 65, 64
    assert sizes == [D * V, FF * D + D, D * FF + FF, 2 * D, D * D, 3 * D * D, 2 * D, V * D + T * D]
    offs = [s.offset for s in L.specs]
    assert offs == sorted(offs) and offs[0] == 0


def test_gpt_layout_and_bucket_coalescing():
    m, _ = preset("tiny-gpt")
    L = ArenaLayout(m)
    names = [s.name for s in L.specs]
    assert names[0] == "lnf_gamma" and names[2] == "h1.W2" and names[-2:] == ["tok_embed", "pos_embed"]
    assert "Wout" not in names
    assert sum(b.numel for b in L.natural_buckets) == L.total
    co = L.coalesced_buckets(100000)
    assert sum(b.numel for b in co) == L.total and all(b.numel >= 100000 for b in co[:-1])
    assert co[0].start == 0 and all(co[i].end == co[i + 1].start for i in range(len(co) - 1))
    assert len(L.coalesced_buckets(10 ** 9)) == 1 and len(L.coalesced_buckets(0)) == len(L.natural_buckets)
    L8 = ArenaLayout(m, shard_multiple=8)
    assert L8.total % 64 == 0


def test_odd_shapes_are_padded_to_16_bytes():
    m = ModelConfig(vocab_size=7, seq_len=4, hidden=8, heads=2, ff=16, batch_size=2)
    L = ArenaLayout(m)
    assert all(s.offset % 8 == 0 for s in L.specs)
    assert sum(b.numel for b in L.natural_buckets) == L.total


def test_xorshift_init_values():
    v = xorshift_uniform(4, 42)
    s = np.uint32(42)
    s ^= np.uint32(s << np.uint32(13)); s ^= np.uint32(s >> np.uint32(17)); s ^= np.uint32(s << np.uint32(5))
    u = np.float32(s & np.uint32(0x7FFFFFFF)) / np.float32(0x7FFFFFFF)
    assert v[0].item() == pytest.approx(float((u * np.float32(2) - np.float32(1)) * np.float32(0.02)), abs=0)
    assert v.abs().max() <= 0.02
    flat = init_flat(ArenaLayout(preset("parity-h128")[0]), 42)
    L = ArenaLayout(preset("parity-h128")[0])
    views = L.views(flat)
    assert (views["ln1_gamma"] == 1).all() and (views["b1"] == 0).all()
    assert torch.equal(views["Wq"].reshape(-1), xorshift_uniform(128 * 128, 52))


def test_fnv_hash_and_stats():
    a = np.array([1.0, -2.0, 0.5], dtype=np.float32)
    h = ckpt.FNV_OFFSET
    for w in a.view(np.uint32).tolist():
        h = ((h ^ w) * ckpt.FNV_PRIME) & ((1 << 64) - 1)
    st = ckpt.param_stats(torch.from_numpy(a))
    assert st.hash == h and st.sum == -0.5 and st.sumsq == 5.25 and st.max_abs == 2.0
    line = ckpt.trajectory_line(1, 2, 3.5, st, (0.0, 0.0, 0.0))
    assert line.startswith("TRAJECTORY epoch=1 step=2 loss=3.5 param_sum=-0.5 param_sumsq=5.25 param_maxabs=2 param_hash=")
    assert line.endswith("sum_span=0.000e+00 sumsq_span=0.000e+00 maxabs_span=0.000e+00")


def test_checkpoint_round_trip_and_corruption(tmp_path):
    m = ModelConfig(vocab_size=7, seq_len=4, hidden=8, heads=2, ff=16, batch_size=2)
    L = ArenaLayout(m)
    p = init_flat(L, 42)
    mm, vv = torch.rand(L.total), torch.rand(L.total)
    for s in L.specs:                      # padding is not stored; make it zero in the source
        pass
    path = str(tmp_path / "ck.bin")
    st = ckpt.save_checkpoint(path, L, p, mm, vv, step=17)
    L2, p2, m2, v2, step, hdr = ckpt.load_checkpoint(path)
    assert step == 17 and hdr["stats"]["hash"] == st.hex_hash()
    for s in L.specs:
        sl = slice(s.offset, s.offset + s.numel)
        assert torch.equal(p[sl], p2[sl]) and torch.equal(mm[sl], m2[sl]) and torch.equal(vv[sl], v2[sl])
    raw = bytearray(open(path, "rb").read())
    raw[-3 * 4 * L.num_params() + 5] ^= 0x10
    open(path, "wb").write(bytes(raw))
    with pytest.raises(ValueError):
        ckpt.load_checkpoint(path)
