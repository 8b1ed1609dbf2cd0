"""Dispatch legality and the verdict stage of the variant search, driven with scripted
timings and checked against what the reference's own hmx_search.py returned on the same
scripts (tests/golden/search_golden.json).  CPU only."""
import json
import math
import os

import pytest

GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "search_golden.json")))
SHAPE = (4096, 4096, 4096)


def order(hm, shape=SHAPE):
    """Variant indices in the search's visiting order for a shape."""
    names = [c["cfg"] for c in hm.gemm_explain(*shape)["candidates"]]
    by_name = {v["name"]: v["variant"] for v in hm.gemm_variants()}
    return [by_name[n] for n in names]


def run_script(hm, timings_abc, canary=(100.0, 99.0, 101.0), canary_reference=100.0, control="a"):
    hm.autotune_cache_clear()
    visit = order(hm)[:3]
    nv = len(hm.gemm_variants())
    table = [(float("inf"),) * 3 for _ in range(nv)]
    for v, t in zip(visit, timings_abc):
        table[v] = tuple(float("inf") if x is None else float(x) for x in t)
    label = {v: l for v, l in zip(visit, "abc")}
    rc, rep = hm.gemm_search_scripted(*SHAPE, table, control=visit["abc".index(control)],
                                      canary=canary, canary_reference=canary_reference)
    champ = label.get(rc) if rc >= 0 else None
    return champ, rep, label


def test_variant_table_and_constants(hm):
    vs = hm.gemm_variants()
    assert len(vs) >= 3
    for v in vs:
        assert v["smem_bytes"] <= 227 * 1024 and v["tmem_cols"] <= 512
        assert v["tiles"][0] % GOLD["constants"]["TILE_EDGE"] == 0


def test_legality_vocabulary(hm):
    # min-rows: M <= 4 is refused before alignment is looked at (HmxTarget.h:100,201)
    assert hm.gemm_variant_verdict(0, GOLD["constants"]["MIN_ROWS"], 4096, 4096) == "min-rows"
    assert hm.gemm_variant_verdict(0, GOLD["constants"]["MIN_ROWS"] + 1, 4096, 4096) == "ok"
    assert hm.gemm_variant_verdict(0, 1, 1023, 4096) == "min-rows"
    assert hm.gemm_variant_verdict(0, 128, 1023, 4096) == "tile-alignment"
    assert hm.gemm_variant_verdict(0, 128, 1024, 4100) == "tile-alignment"
    assert hm.gemm_variant_verdict(0, 128, 1024, 4104) == "ok"
    with pytest.raises(ValueError):
        hm.gemm_variant_verdict(99, 128, 128, 128)


def test_explain_names_plan_and_reason(hm):
    e = hm.gemm_explain(1024, 1024, 1024)
    assert e["plan"] == "tcgen05" and e["reference_plan"] == "hmx" and e["variant"] >= 0
    e = hm.gemm_explain(1, 11008, 4096)
    assert e["plan"] == "cuda-core" and e["reference_plan"] == "hvx" and e["reason"] == "min-rows"
    models = [c["model_clocks"] for c in hm.gemm_explain(8192, 8192, 8192)["candidates"]]
    assert models == sorted(models)  # visited by modelled lower bound


@pytest.mark.parametrize("name", sorted(GOLD["rounds"]))
def test_champion_round_matches_reference(hm, name):
    g = GOLD["rounds"][name]
    canary = tuple(g["canary"]) if "canary" in g else (100.0, 99.0, 101.0)
    champ, rep, _ = run_script(hm, g["timings"], canary=canary)
    assert champ == g["champion"]
    assert rep["round_verdict"] == g["round_verdict"]
    assert rep["champion_significant"] == g["champion_significant"]
    assert [c["outcome"] for c in rep["comparisons"]] == g["outcomes"]
    assert len(rep["unmeasured"]) >= len(g["unmeasured"])
    assert rep["gate"]["form"] == "max(3xCV, 15%)"


@pytest.mark.parametrize("name", sorted(GOLD["canary"]))
def test_canary_verdict_matches_reference(hm, name):
    g = GOLD["canary"][name]
    m = g["metrics"]
    canary = None if m is None else (m["q50_pcyc"], m["q20_pcyc"], m["q80_pcyc"])
    ref = float("nan") if g["reference"] is None else g["reference"]
    _, rep, _ = run_script(hm, [(100, 99, 101)] * 3, canary=canary, canary_reference=ref)
    assert rep["canary"]["status"] == g["status"]
    assert rep["canary"]["healthy"] == g["healthy"]
    assert (rep["round_verdict"] == "valid") == g["healthy"]


def test_gate_values_match_reference(hm):
    # challenger faster by delta against an incumbent with spread cv: takeover iff delta > gate
    for cv, gate in GOLD["champion_gate"]:
        if cv != cv or gate >= 0.9:  # a gate of 150% cannot be cleared by a positive time
            continue
        base = 1000.0
        spread = cv * base
        inc = (base, base - spread / 2, base + spread / 2)
        for delta, want in ((gate * 1.02, "takeover"), (gate * 0.98, "kept")):
            ch = base * (1 - delta)
            _, rep, _ = run_script(hm, [inc, (ch, ch, ch), (1e9, 1e9, 1e9)])
            assert rep["comparisons"][0]["outcome"] == want, (cv, gate, delta)
            assert rep["comparisons"][0]["gate_pct"] == pytest.approx(100 * gate, rel=1e-4)


def test_void_round_does_not_enter_the_cache(hm, tmp_path):
    hm.autotune_cache_clear()
    g = GOLD["rounds"]["void_round"]
    run_script(hm, g["timings"], canary=tuple(g["canary"]))
    p = tmp_path / "cache.json"
    hm.autotune_cache_save(str(p))
    assert json.load(open(p))["entries"] == []


def test_cache_roundtrip_and_dispatch_uses_it(hm, tmp_path):
    hm.autotune_cache_clear()
    visit = order(hm)
    champ, rep, label = run_script(hm, GOLD["rounds"]["chain"]["timings"])
    assert champ == "c"
    e = hm.gemm_explain(*SHAPE)
    assert e["reason"] == "autotune cache" and e["variant"] == visit[2]
    p = tmp_path / "cache.json"
    hm.autotune_cache_save(str(p))
    entries = json.load(open(p))["entries"]
    assert len(entries) == 1 and entries[0]["variant"] == visit[2]
    assert "4096|4096|4096" in entries[0]["key"]
    hm.autotune_cache_clear()
    assert hm.gemm_explain(*SHAPE)["reason"] == "modelled lower bound"
    hm.autotune_cache_load(str(p))
    assert hm.gemm_explain(*SHAPE)["reason"] == "autotune cache"
    # another shape is not affected
    assert hm.gemm_explain(2048, 2048, 2048)["reason"] == "modelled lower bound"
    hm.autotune_cache_clear()


def test_failed_candidates_score_inf_not_abort(hm):
    champ, rep, _ = run_script(hm, [(100, 99, 101), (float("nan"),) * 3, (-5, -5, -5)])
    assert champ == "a" and len(rep["unmeasured"]) >= 2
    assert all(math.isfinite(c["q50_us"]) or c["q50_us"] is None for c in rep["candidates"]
               if c["q50_us"] is not None)
