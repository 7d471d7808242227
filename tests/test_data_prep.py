"""Shard writer of the data-preparation script (no tokenizer or network needed)."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "data", f"{name}.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_shards_split_documents_across_boundaries(tmp_path):
    prep = _load("prepare_fineweb")
    from dion_b200.models.data import _read_shard

    def fake_tokenize(doc):  # "document" = its length; eot modelled as 0
        n = int(doc)
        return np.concatenate([[0], np.arange(1, n + 1)]).astype(np.uint16)

    docs = ["7", "5", "12", "3"]
    files = prep.build_shards(docs, str(tmp_path), shard_size=10, workers=1,
                              tokenize=fake_tokenize)
    names = [os.path.basename(f) for f in files]
    assert names[0] == "fineweb_val_000000.bin" and names[1] == "fineweb_train_000001.bin"
    got = np.concatenate([_read_shard(f) for f in files])
    want = np.concatenate([fake_tokenize(d) for d in docs])
    assert np.array_equal(got, want)
    assert all(len(_read_shard(f)) == 10 for f in files[:-1])


def test_cached_shard_names():
    dl = _load("download_cached")
    names = list(dl.shard_names("fineweb", 2))
    assert names == ["fineweb_val_000000.bin", "fineweb_train_000001.bin",
                     "fineweb_train_000002.bin"]
    assert set(dl.DATASETS) == {"fineweb10B", "fineweb100B", "finewebedu10B"}
