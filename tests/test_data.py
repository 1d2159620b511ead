import json

import numpy as np
import pytest
import torch

from idrak_b200 import data as D


def _ds(n=103):
    return D.TensorDataset(torch.arange(n, dtype=torch.float32)[:, None], torch.arange(n))


def test_shards_tile_the_single_process_batches():
    world, bs = 4, 5
    single = D.DataLoader(_ds(), batch_size=bs * world, shuffle=True, seed=7)
    big = [b[1] for b in single]
    shards = []
    for r in range(world):
        ld = D.DataLoader(_ds(), batch_size=bs, shuffle=True, seed=7)
        shards.append([b[1] for b in ld.shard(r, world)])
    for k, whole in enumerate(big):
        parts = [shards[r][k] for r in range(world) if k < len(shards[r])]
        merged = torch.stack([p for p in parts if len(p) == len(parts[0])]).t().reshape(-1) if len({len(p) for p in parts}) == 1 \
            else torch.cat(parts).sort().values
        assert sorted(merged.tolist()) == sorted(whole.tolist())
        assert whole[0::world].tolist() == shards[0][k].tolist()        # rank r takes positions k * world + r
    assert sum(len(b) for s in shards for b in s) == 103
    # a second epoch draws a different order, the same on every rank
    a = D.DataLoader(_ds(), batch_size=8, shuffle=True, seed=1)
    e0 = torch.cat([b[1] for b in a]).tolist()
    e1 = torch.cat([b[1] for b in a]).tolist()
    assert e0 != e1 and sorted(e0) == sorted(e1) == list(range(103))
    assert len(D.DataLoader(_ds(), batch_size=10, drop_last=True)) == 10 and len(D.DataLoader(_ds(), batch_size=10)) == 11


def test_step_shares_follow_a_changing_group():
    world, bs = 3, 4
    ld = [D.DataLoader(_ds(60), batch_size=bs, shuffle=True, seed=3) for _ in range(world)]
    ref = D.DataLoader(_ds(60), batch_size=bs * world, shuffle=True, seed=3)
    whole = [b[1].tolist() for b in ref]
    step = [0]
    # rank 2 sits out every second step
    def place_for(r):
        def place():
            k = step[0]
            if k % 2 == 1:
                return None if r == 2 else (r, 2)
            return (r, 3)
        return place
    its = [ld[r].step_shares(world, place_for(r)) for r in range(world)]
    for k in range(len(whole)):
        step[0] = k
        got = [next(it) for it in its]
        if k % 2 == 1:
            assert got[2] is None
        seen = sorted(v for g in got if g is not None for v in g[1].tolist())
        assert seen == sorted(whole[k])                   # the step's samples are dealt among those taking part
    for it in its:
        with pytest.raises(StopIteration):
            next(it)


def test_bucketing_prefetch_transforms_and_ragged_collate():
    lengths = np.random.default_rng(0).integers(1, 40, 200)

    class Ragged(D.Dataset):
        def __len__(self):
            return 200

        def __getitem__(self, i):
            return (torch.full((int(lengths[i]),), i),)

    plain = D.DataLoader(Ragged(), batch_size=8, shuffle=True, seed=1)
    bucketed = D.DataLoader(Ragged(), batch_size=8, shuffle=True, seed=1, bucket_by=lambda i: int(lengths[i]), bucket_size=25,
                            prefetch=2)
    def waste(loader):
        pad = tot = 0
        ids = []
        for x, n in loader:
            pad += x.shape[0] * x.shape[1] - int(n.sum())
            tot += x.shape[0] * x.shape[1]
            ids += x[:, 0].tolist()
        assert sorted(ids) == list(range(200))
        return pad / tot
    assert waste(bucketed) < 0.5 * waste(plain)
    seen = []
    ld = D.DataLoader(_ds(10), batch_size=5, transforms=[lambda s: (s[0] * 2, s[1]), lambda s, epoch, index: (seen.append((epoch, index)), s)[1]])
    out = torch.cat([b[0] for b in ld])
    assert out[:, 0].tolist() == [2.0 * i for i in range(10)] and seen[0] == (0, 0) and len(seen) == 10

    class Broken(D.Dataset):
        def __len__(self):
            return 4

        def __getitem__(self, i):
            raise RuntimeError("bad sample")
    with pytest.raises(RuntimeError, match="bad sample"):
        list(D.DataLoader(Broken(), batch_size=2, prefetch=1))
    a, b = _ds(100).split(0.8, seed=2)
    assert len(a) == 80 and len(b) == 20 and not set(a.indices.tolist()) & set(b.indices.tolist())
    w = D.TokenWindows(np.arange(1000, dtype=np.uint16), 64)
    x, y = w[3]
    assert len(w) == 15 and x[0] == 192 and torch.equal(x[1:], y[:-1])


def test_readers_and_row_operations(tmp_path):
    rows = [{"text": f"row number {i} " + "word " * (i % 7), "label": i % 3} for i in range(50)]
    p = tmp_path / "a.jsonl"
    assert D.write_jsonl(rows, str(p)) == 50
    assert list(D.read_records(str(p))) == rows
    (tmp_path / "b.json").write_text(json.dumps({"data": rows[:5]}))
    assert list(D.read_json(str(tmp_path / "b.json"))) == rows[:5]
    (tmp_path / "c.tsv").write_text("a\tb\n1\tx\n2\ty\n")
    assert list(D.read_records(str(tmp_path / "c.tsv"))) == [{"a": "1", "b": "x"}, {"a": "2", "b": "y"}]
    (tmp_path / "d.txt").write_text("one\n\ntwo lines\nhere\n")
    assert [r["text"] for r in D.read_text(str(tmp_path / "d.txt"), by="paragraph")] == ["one", "two lines\nhere"]
    import pyarrow as pa
    import pyarrow.parquet as pq
    pq.write_table(pa.table({"text": ["x", "y"], "n": [1, 2]}), str(tmp_path / "e.parquet"))
    assert list(D.read_records(str(tmp_path / "e.parquet"))) == [{"text": "x", "n": 1}, {"text": "y", "n": 2}]
    assert len(list(D.read_records(str(tmp_path)))) == 50 + 5 + 2 + 3 + 2
    with pytest.raises(OSError, match="network"):
        list(D.read_records("https://example.com/x.jsonl"))
    with pytest.raises(ValueError, match="a.jsonl:1"):
        (tmp_path / "bad").mkdir()
        (tmp_path / "bad" / "a.jsonl").write_text("{nope\n")
        list(D.read_records(str(tmp_path / "bad" / "a.jsonl")))
    src = tmp_path / "code"
    (src / "pkg").mkdir(parents=True)
    (src / ".git").mkdir()
    (src / "pkg" / "m.py").write_text("print(1)\n")
    (src / ".git" / "x.py").write_text("hidden\n")
    assert [r["path"] for r in D.read_code(str(src))] == ["pkg/m.py"]

    kept = list(D.filter_rows(rows, lambda r: r["label"] == 0))
    assert len(kept) == 17
    assert [r["n"] for r in D.map_rows(rows[:3], lambda r: {"n": len(r["text"])} if r["label"] else None)] == [len(rows[1]["text"]), len(rows[2]["text"])]
    s1, s2 = list(D.shuffle_rows(rows, seed=4)), list(D.shuffle_rows(rows, seed=4, buffer=8))
    assert s1 != rows and sorted(map(str, s1)) == sorted(map(str, rows)) == sorted(map(str, s2))
    dup = rows + [{"text": "ROW   number 3 word word word "}, dict(rows[10])]
    assert len(list(D.dedupe(dup))) == 50
    base = "the quick brown fox jumps over the lazy dog and runs far away into the deep dark forest tonight"
    near = [{"text": base}, {"text": base + " again"}, {"text": "completely different words appear in this other sentence right here"}]
    assert len(list(D.dedupe(near))) == 3 and len(list(D.dedupe(near, near=True, threshold=0.7))) == 2
    a, b = D.split_rows(rows, 0.9, seed=1)
    assert len(a) == 45 and len(b) == 5
    m = list(D.mix([[{"s": 0}] * 30, [{"s": 1}] * 10], weights=[3, 1], seed=0))
    assert len(m) == 40 and sum(r["s"] for r in m[:20]) < 10
    assert len(list(D.mix([[{"s": 0}] * 30, [{"s": 1}] * 2], seed=0, stop="first"))) < 32


def test_csv_tables_and_scalers(tmp_path):
    p = tmp_path / "houses.csv"
    p.write_text("area,rooms,city,price\n100,3,A,10\n150,4,B,20\n80,2,A,8\n")
    ds, feats, cats = D.csv_dataset(str(p), targets=["price"])
    assert feats == ["area", "rooms", "city"] and cats == {"city": ["A", "B"]}
    x, y = ds[1]
    assert x.tolist() == [150.0, 4.0, 1.0] and y.tolist() == [20.0]
    with pytest.raises(KeyError, match="columns: area"):
        D.csv_dataset(str(p), targets=["cost"])
    for scaler in (D.StandardScaler().fit(ds.features), D.MinMaxScaler().fit(ds.features)):
        z = scaler.transform(ds.features)
        assert torch.allclose(scaler.inverse(z), ds.features, atol=1e-4)
        scaler.save(str(tmp_path / "s.txt"))
        again = D.load_scaler(str(tmp_path / "s.txt"))
        assert type(again) is type(scaler) and torch.allclose(again.transform(ds.features), z)
    assert abs(D.StandardScaler().fit(ds.features).transform(ds.features).mean().item()) < 1e-6
