"""Host-side helpers for a data-parallel command-line trainer (no GPU needed): rank and world from the launcher's
environment, and this rank's share of the samples train_load_data left in the state (src/train.c:812)."""
import ctypes as C

import numpy as np


def lib():
    from seraph_b200 import api, build
    build.build()
    return api.load()


def test_rank_and_world_from_the_environment(monkeypatch):
    L = lib()
    r, w = C.c_int(-1), C.c_int(-1)
    for k in ("SERAPH_DP_RANK", "SERAPH_DP_WORLD", "RANK", "WORLD_SIZE"):
        monkeypatch.delenv(k, raising=False)
    assert L.seraph_dp_env(C.byref(r), C.byref(w)) == 0 and (r.value, w.value) == (0, 1)
    monkeypatch.setenv("RANK", "3"); monkeypatch.setenv("WORLD_SIZE", "8")
    assert L.seraph_dp_env(C.byref(r), C.byref(w)) == 0 and (r.value, w.value) == (3, 8)
    monkeypatch.setenv("SERAPH_DP_RANK", "1"); monkeypatch.setenv("SERAPH_DP_WORLD", "2")       # the library's own names win
    assert L.seraph_dp_env(C.byref(r), C.byref(w)) == 0 and (r.value, w.value) == (1, 2)
    monkeypatch.setenv("SERAPH_DP_RANK", "2")
    assert L.seraph_dp_env(C.byref(r), C.byref(w)) == 1                                         # rank outside the world


def test_sample_shards_are_disjoint_equal_and_keep_sample_ends():
    L = lib()
    lens = np.random.default_rng(5).integers(1, 40, 23)
    offs0 = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    total = int(lens.sum())
    tokens = np.arange(total)
    seen = []
    for world in (1, 2, 4, 8):
        per = len(lens) // world
        covered = []
        for rank in range(world):
            offs, n, nt = offs0.copy(), C.c_int(len(lens)), C.c_int(total)
            first = L.seraph_dp_shard_samples(offs.ctypes.data, C.byref(n), C.byref(nt), rank, world)
            assert first == rank * per and n.value == per
            # the trainer's rule: sample i is [offs[i], offs[i+1]) and the last one ends at num_train_tokens
            for i in range(per):
                s = offs[i]
                e = offs[i + 1] if i + 1 < per else nt.value
                assert (s, e) == (offs0[first + i], offs0[first + i] + lens[first + i])
                covered.append((int(s), int(e)))
        assert len(set(covered)) == per * world                       # disjoint, same count on every rank
        seen.append(covered)
    assert L.seraph_dp_shard_samples(None, None, None, 0, 2) == -1
    offs, n, nt = offs0.copy(), C.c_int(len(lens)), C.c_int(total)
    assert L.seraph_dp_shard_samples(offs.ctypes.data, C.byref(n), C.byref(nt), 2, 2) == -1
    assert tokens.size == total
