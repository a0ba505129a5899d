"""The performance-history CSV of bench.py (--csv with --generate / --update / --compare), modelled on the reference's
benchmark driver (benchmark/README.md:84-103): records keyed by device, operator, dtype and shape; an update needs
more than 5 % improvement; compare changes nothing."""
from mcoplib_b200 import perf_csv as P


def _rec(op, us, gbs=5000.0, shape="tokens=1024"):
    return P.make_record("B200", op, "bf16", shape, 10, us, gbs, 6537.0)


def test_generate_adds_only_new_keys(tmp_path):
    f = str(tmp_path / "hist" / "perf.csv")
    r = P.apply(f, [_rec("chain5/norm_quant", 2000.0), _rec("chain5/gather", 1800.0)], "generate")
    assert [e["action"] for e in r] == ["added", "added"]
    rows = P.load(f)
    assert len(rows) == 2 and rows[0]["Op"] == "chain5/norm_quant" and rows[0]["BWUtil (%)"] == "76.49"
    r = P.apply(f, [_rec("chain5/norm_quant", 1000.0), _rec("chain5/scatter", 1300.0)], "generate")
    assert [e["action"] for e in r] == ["kept", "added"]
    rows = P.load(f)
    assert len(rows) == 3 and rows[0]["GPU Time (us)"] == "2000.000"      # an existing record is not touched by generate


def test_update_needs_more_than_five_percent(tmp_path):
    f = str(tmp_path / "perf.csv")
    P.apply(f, [_rec("op", 100.0)], "generate")
    assert P.apply(f, [_rec("op", 96.0)], "update")[0]["action"] == "kept" and P.load(f)[0]["GPU Time (us)"] == "100.000"
    assert P.apply(f, [_rec("op", 110.0)], "update")[0]["action"] == "kept"
    e = P.apply(f, [_rec("op", 94.0, 5300.0)], "update")[0]
    assert e["action"] == "updated" and abs(e["change"] + 0.06) < 1e-9
    assert P.load(f)[0]["GPU Time (us)"] == "94.000" and P.load(f)[0]["GlobalMem BW (GB/s)"] == "5300.0"
    # another shape is another record
    assert P.apply(f, [_rec("op", 50.0, shape="tokens=2048")], "update")[0]["action"] == "added" and len(P.load(f)) == 2


def test_compare_changes_nothing_and_reports(tmp_path):
    f = str(tmp_path / "perf.csv")
    P.apply(f, [_rec("a", 100.0)], "generate")
    before = open(f).read()
    r = P.apply(f, [_rec("a", 80.0), _rec("b", 10.0)], "compare")
    assert [e["action"] for e in r] == ["compared", "missing"] and abs(r[0]["change"] + 0.2) < 1e-9
    assert open(f).read() == before
    text = P.format_report(r)
    assert "old 100.000 us  new 80.000 us  (-20.0 %)" in text and "missing" in text
