"""The collectives' launch-shape table: lookup by size bucket, sub-tables per buffer kind,
environment override, and the table builder used by the tuner."""
import json

from commbench_b200.ops import tuning


def test_make_rows_puts_boundaries_at_geometric_means():
    rows = tuning.make_rows([(1 << 20, {"blocks": 8}), (16 << 20, {"blocks": 64}),
                             (256 << 20, {"blocks": 148})])
    assert rows[0][0] == 4 << 20 and rows[1][0] == 64 << 20 and rows[2][0] is None
    assert [r[1]["blocks"] for r in rows] == [8, 64, 148]


def test_lookup_prefers_the_kind_sub_table_and_handles_missing(tmp_path, monkeypatch):
    path = tmp_path / "t.json"
    tuning.merge_into(path, 8, {
        "all_reduce": tuning.make_rows([(1 << 20, {"algo": "oneshot"}),
                                        (64 << 20, {"algo": "nvls", "blocks": 96, "unroll": 8})]),
        "all_reduce@staged": tuning.make_rows([(64 << 20, {"algo": "twoshot_push"})]),
    })
    monkeypatch.setenv("CB200_TUNE_TABLE", str(path))
    tuning.reload()
    assert tuning.lookup("all_reduce", 8, 4096)["algo"] == "oneshot"
    assert tuning.lookup("all_reduce", 8, 32 << 20) == {"algo": "nvls", "blocks": 96, "unroll": 8}
    assert tuning.lookup("all_reduce", 8, 1 << 30)["algo"] == "nvls"          # open-ended last row
    assert tuning.lookup("all_reduce", 8, 4096, "staged")["algo"] == "twoshot_push"
    assert tuning.lookup("all_reduce", 8, 4096, "symmetric")["algo"] == "oneshot"
    assert tuning.lookup("all_reduce", 4, 4096) == {}                          # no such world
    assert tuning.lookup("all_gather", 8, 4096) == {}                          # no such op
    # a second world size merges into the same file
    tuning.merge_into(path, 2, {"all_gather": tuning.make_rows([(1 << 20, {"blocks": 32})])})
    table = json.loads(path.read_text())
    assert set(table["world"]) == {"2", "8"}
    assert tuning.lookup("all_gather", 2, 123)["blocks"] == 32
    monkeypatch.setenv("CB200_TUNE_TABLE", "off")
    assert tuning.lookup("all_reduce", 8, 4096) == {}
    monkeypatch.delenv("CB200_TUNE_TABLE")
    tuning.reload()


def test_unreadable_table_is_ignored(tmp_path, monkeypatch):
    bad = tmp_path / "bad.json"
    bad.write_text("{not json")
    monkeypatch.setenv("CB200_TUNE_TABLE", str(bad))
    tuning.reload()
    assert tuning.lookup("all_reduce", 8, 4096) == {}
    monkeypatch.delenv("CB200_TUNE_TABLE")
    tuning.reload()


def test_plan_all_reduce_falls_back_without_multicast(tmp_path, monkeypatch):
    from commbench_b200.ops import collectives as coll

    class Ctx:
        world, has_multicast = 8, False

    path = tmp_path / "t.json"
    tuning.merge_into(path, 8, {"all_reduce": tuning.make_rows(
        [(64 << 20, {"algo": "nvls", "blocks": 96, "unroll": 8})])})
    monkeypatch.setenv("CB200_TUNE_TABLE", str(path))
    tuning.reload()
    plan = coll.plan_all_reduce(Ctx, 64 << 20, True)
    assert plan["algo"] == "twoshot" and plan["blocks"] is None
    Ctx.has_multicast = True
    assert coll.plan_all_reduce(Ctx, 64 << 20, True) == {"algo": "nvls", "blocks": 96, "unroll": 8}
    assert coll.plan_all_reduce(Ctx, (64 << 20) + 8, True)["algo"] != "nvls"   # not 16-byte sized
    monkeypatch.delenv("CB200_TUNE_TABLE")
    tuning.reload()


def test_tuner_grid_candidates_are_bounded():
    from commbench_b200.ops.tune import _grid_candidates

    assert _grid_candidates(8192) == [1]                      # never less than 8 KB per CTA
    assert max(_grid_candidates(1 << 30)) == 128              # never all 148 SMs
    assert min(_grid_candidates(128 << 20)) >= 64             # never more than 2 MB per CTA
    for share in (65536, 1 << 20, 32 << 20):
        g = _grid_candidates(share)
        assert g == sorted(g) and len(set(g)) == len(g)
