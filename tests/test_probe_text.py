"""Text-level probe generators: determinism, lengths, the facts in place, the stored form and its checks, the build script."""

import gzip
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from gdn_hybrid_architecture_ideas_b200.eval import probe_text as T

ROOT = Path(__file__).resolve().parent.parent
WORDS = "the of and a to in is that it was for on are as with his they at be this from have or by one had not but what all were when we there can an your which their said if do will each about how up out them then she many some so these would other into has more her two like him see time could no make than first been its who now people my made over did down only way find use may water long little very after words called just where most know".split()


def docs(n=60, seed=0):
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n):
        sents = []
        for _ in range(int(rng.integers(30, 60))):
            w = [WORDS[i] for i in rng.integers(len(WORDS), size=int(rng.integers(6, 16)))]
            sents.append(" ".join(w).capitalize() + ".")
        out.append(" ".join(sents))
    return out


COUNT = lambda text: len(text.encode("utf-8")) // 4          # a stand-in length measure: four bytes per token


@pytest.fixture(scope="module")
def pool():
    return T.DocPool(docs())


def test_a_needle_item_has_its_length_its_sentence_at_the_depth_and_is_reproducible(pool):
    a = T.uuid_needle(pool, COUNT, 2048, 0.3, 5)
    b = T.uuid_needle(pool, COUNT, 2048, 0.3, 5)
    assert a.to_json() == b.to_json()
    assert T.uuid_needle(pool, COUNT, 2048, 0.3, 6).answer != a.answer
    n = COUNT(a.context + a.answer)
    assert (1 - T.LENGTH_SLACK) * 2048 <= n <= 2048
    name, value = a.meta["name"], a.answer.strip()
    assert a.context.count(T.needle_sentence(name, value)) == 1 and a.context.endswith(T.needle_question(name))
    at = a.context.index(value) / len(a.context)
    assert abs(at - 0.3) < 0.08
    assert T.question_text(a) == T.needle_question(name)
    assert T.TextItem.from_json(json.loads(json.dumps(a.to_json()))).to_json() == a.to_json()


def test_multikey_asks_one_of_n_distinct_needles(pool):
    it = T.multikey(pool, COUNT, 2048, 4, 1)
    sentences = [m for m in it.context.split(". ") if "The access code for" in m and "What is" not in m]
    assert len(sentences) >= 4 and it.context.count(it.answer.strip()) == 1
    assert len(it.meta["needle_offsets"]) == 4 and 0 <= it.meta["asked"] < 4


def test_needle_at_a_token_distance(pool):
    it = T.needle_at_distance(pool, COUNT, 4096, 1024, 2, tol=96)
    at = it.context.rfind(it.answer.strip())
    assert abs(COUNT(it.context[at:]) - 1024) <= 96 and it.cell["distance"] == 1024
    same = T.needle_at_distance(pool, COUNT, 4096, 2048, 2, tol=96)
    assert same.answer == it.answer and same.meta["name"] == it.meta["name"]          # the item keeps its name and value at every distance


def test_path_copy_grids():
    one = T.path_copy(8, (8, 1, 1), "deep", 3)
    lines = [ln for ln in one.context.splitlines() if " -> " in ln]
    paths = [ln.split(" -> ")[1] for ln in lines]
    assert len(paths) == 8 and len(set(paths)) == 8 and one.answer.strip() in paths and one.context.endswith(f"class {one.meta['name']} ->")
    parts = [p.split("/") for p in paths]
    differing = [i for i in range(len(parts[0])) if len({p[i] for p in parts}) > 1]
    assert len(differing) == 1                                           # one directory decides the path
    near = T.path_copy(12, (2, 3, 4), "shallow", 0)
    assert len({ln.split(" -> ")[1] for ln in near.context.splitlines() if " -> " in ln}) == 12
    with pytest.raises(ValueError):
        T.path_copy(12, (2, 2, 2), "deep", 0)


@pytest.mark.parametrize("hops", [0, 3, 8])
def test_depth_items_execute_to_their_answer_and_balance_the_rank(hops):
    ranks = set()
    for i in range(6):
        it = T.depth(hops, i)
        scope = {}
        exec(it.context + it.answer + "\nmain()", scope)                  # the program is valid Python and its assert holds
        wrong = next(c for c in it.candidates if c != it.answer)
        with pytest.raises(AssertionError):
            exec(it.context + wrong + "\nmain()", {})
        assert it.candidates[it.gold] == it.answer and len(set(it.meta["assigned"])) == T.CHAINS
        literal_lines = [ln.strip() for ln in it.context.splitlines() if ln.strip()[-1:].isdigit() and " = " in ln]
        asked_first = next(k for k, ln in enumerate(literal_lines) if ln.endswith(f"= {it.answer}"))
        assert asked_first == it.meta["rank"] == i % T.CHAINS
        ranks.add(asked_first)
    assert ranks == set(range(T.CHAINS))


@pytest.mark.parametrize("probe", ["mf_chain", "mf_concat"])
def test_multifact_answers_need_every_fact(pool, probe):
    it = T.multifact(probe, pool, COUNT, 4096, 4, 1)
    pieces = it.meta["pieces"]
    assert "".join(p for p, _ in pieces) == it.answer and sum(1 for _, f in pieces if f) == 4
    for text, is_fact in pieces:
        if is_fact:
            assert it.context.count(text.strip()) >= 1
    assert it.group["layout"] == T.LAYOUTS[1]
    offs = it.meta["fact_offsets"]
    lo, hi = T.LAYOUT_SPAN["front"]
    assert all(lo - 0.05 <= o <= hi + 0.1 for o in offs), offs
    if probe == "mf_chain":
        names = [p.strip() for p, f in pieces if f]
        assert all(f"is {n}." in it.context for n in names)


def test_stored_form_and_checks(pool):
    enc = lambda s: list(s.encode("utf-8"))
    rec = T.encode_item(T.uuid_needle(pool, COUNT, 1024, 0.5, 0), enc)
    assert rec["ids"][rec["answer_start"]:] == enc(" " + bytes(rec["ids"][rec["answer_start"] + 1:]).decode()) and rec["checks"] == {"clean_boundary": True, "answer_once": True}
    assert rec["question_tokens"] > 10 and rec["kind"] == "uuid_needle" and rec["cell"] == "length=1024"
    d = T.encode_item(T.depth(2, 0), enc)
    assert d["checks"]["single_token_candidates"] and d["candidates"][d["gold"]] == d["ids"][d["answer_start"]:]
    mf = T.encode_item(T.multifact("mf_concat", pool, COUNT, 2048, 2, 0), enc)
    assert mf["checks"]["pieces_add_up"] and [f for _, f in mf["pieces"]] == [True, False, True]


def test_build_script_writes_text_sets_and_manifests(tmp_path):
    src = tmp_path / "docs.jsonl.gz"
    with gzip.open(src, "wt") as f:
        for i, d in enumerate(docs(40, seed=3)):
            f.write(json.dumps({"id": i, "text": d}) + "\n")
    out = tmp_path / "set"
    r = subprocess.run([sys.executable, str(ROOT / "scripts/build_text_probes.py"), "--out", str(out), "--tokenizer", "bytes=bytes", "--docs", str(src),
                        "--probes", "uuid_needle,depth,mf_chain", "--lengths", "4096", "--per-cell", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    manifest = json.loads((out / "manifest.json").read_text())
    assert manifest["failed_checks"] == 0 and manifest["probes"] == {"uuid_needle": 5, "depth": 9, "mf_chain": 3}
    stored = torch.load(out / "bytes" / "uuid_needle.pt", weights_only=False)
    assert len(stored["probes"]) == 5 and all(3900 <= p["length"] <= 4096 for p in stored["probes"])
    with gzip.open(out / "text" / "depth.jsonl.gz", "rt") as f:
        assert len([T.TextItem.from_json(json.loads(x)) for x in f]) == 9


def test_text_sets_are_scored_by_the_probe_scorer(tmp_path):
    """A stored text-level set goes through scripts/eval_probes.py: cells by name, exact match, the ten-way choice of depth."""
    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    model = C.tiny_full_config()
    model.vocab_size = 256
    cfg = C.TrainConfig(model=model, data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 1, 0, False, "cpu"
    Trainer(cfg, tmp_path / "run").fit()
    out = tmp_path / "set"
    r = subprocess.run([sys.executable, str(ROOT / "scripts/build_text_probes.py"), "--out", str(out), "--tokenizer", "bytes=bytes",
                        "--probes", "path_copy,depth", "--per-cell", "1"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    for probe, cells in (("depth", len(T.HOPS)), ("path_copy", 2 * len(T.PATH_CELLS))):
        res = tmp_path / f"{probe}.json"
        r = subprocess.run([sys.executable, str(ROOT / "scripts/eval_probes.py"), "--checkpoint", str(tmp_path / "run"), "--set", str(out / "bytes" / f"{probe}.pt"),
                            "--device", "cpu", "--batch-size", "2", "--out", str(res)], capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        table = json.loads(res.read_text())["probes"]
        assert len(table) == cells and all(0.0 <= c["exact"] <= 1.0 and c["n"] == 1 for c in table.values())
        if probe == "depth":
            assert all("choice_acc" in c for c in table.values()) and "hops=3@depth" not in table and any(k.startswith("depth@hops=") for k in table)


def test_twohop_variants_share_a_haystack_and_differ_in_their_links(pool):
    items = {it.cell["variant"]: it for it in T.twohop(pool, COUNT, 4096, "near", 3, "word", 2)}
    assert set(items) == set(T.TWOHOP_VARIANTS)
    two, one, link, shuf, swap = (items[v] for v in T.TWOHOP_VARIANTS)
    head, bridge, code = two.meta["head"], two.meta["bridge"], two.answer.strip()
    assert bridge not in two.context.split(T.JOIN)[-1] and one.answer == two.answer == shuf.answer == swap.answer and link.answer.strip() == bridge
    assert f"The supervisor of {head} is {bridge}." in two.context and f"The access code for {bridge} is {code}." in two.context
    assert f"The supervisor of {head} is {bridge}." not in shuf.context and f"The access code for {bridge} is {code}." in shuf.context
    assert f"The supervisor of {head} is {bridge}." not in swap.context and swap.context.count(f"is {bridge}.") == 1      # another head now names this bridge
    codes = two.meta["codes"]
    assert len({c[0] for c in codes}) == 4 and swap.meta["followed"].strip() == codes[1]
    body = lambda it: it.context.rsplit(T.JOIN, 1)[0]
    strip = lambda t: [ln for ln in t.split(". ") if "supervisor of" not in ln]
    assert strip(body(two)) == strip(body(swap)) == strip(body(shuf))               # only link sentences differ between the variants
    ranks = set()
    for i in range(8):
        it = T.twohop(pool, COUNT, 2048, "adjacent", 3, "uuid", i)[0]
        order_in_text = sorted(it.meta["codes"], key=lambda c: it.context.index(c))
        ranks.add((order_in_text.index(it.meta["codes"][0]), it.group["order"]))
        assert it.meta["codes"][0][0] in "abcdef"
    assert ranks == {(r, o) for r in range(4) for o in ("AB", "BA")}
    s = T.twohop_summary({"twohop": [1, 1, 0, 1], "swapped": [0, 0, 0, 1], "onehop": [1, 1, 1, 1]})
    assert s["follows_link"] == 0.5 and s["hop_cost"] == 0.25


def test_variable_tracking_has_two_chains_and_asks_for_one(pool):
    it = T.var_track(pool, COUNT, 2048, 3)
    asked, other = it.meta["chains"]
    assert it.answer == " " + " ".join(asked) and len(asked) == len(other) == T.VT_HOPS + 1
    stmts = [m for m in it.context.split(". ") if m.startswith("VAR ") or " VAR " in m[:12]]
    text = it.context
    assert text.index(f"VAR {asked[0]} = {it.meta['numbers'][0]}.") < text.index(f"VAR {asked[1]} = VAR {asked[0]}.") < text.index(f"VAR {asked[3]} = VAR {asked[2]}.")
    assert f"VAR {other[0]} = {it.meta['numbers'][1]}." in text and it.meta["numbers"][0] != it.meta["numbers"][1]
    assert text.count("VAR ") >= 2 * (T.VT_HOPS + 1) and (1 - T.LENGTH_SLACK) * 2048 <= COUNT(text + it.answer) <= 2048
    assert T.var_track(pool, COUNT, 2048, 3).to_json() == it.to_json()


def test_pcr_preset_writes_retrieval_and_copy_sets(tmp_path):
    src = tmp_path / "docs.jsonl"
    src.write_text("".join(json.dumps({"id": i, "text": d}) + "\n" for i, d in enumerate(docs(40, seed=4))))
    out = tmp_path / "pcr"
    r = subprocess.run([sys.executable, str(ROOT / "scripts/build_text_probes.py"), "--out", str(out), "--tokenizer", "bytes=bytes", "--docs", str(src),
                        "--preset", "pcr", "--per-cell", "1", "--copy-lengths", "16,32", "--copy-per-length", "2"], capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    m = json.loads((out / "manifest.json").read_text())
    assert m["probes"]["uuid_needle"] == 15 and m["probes"]["multikey"] == 6 and m["probes"]["vt"] == 3 and m["probes"]["pcr_copy3"] == 4
    copy2 = torch.load(out / "bytes" / "pcr_copy2.pt", weights_only=False)["probes"]
    assert copy2[0]["ids"][:16] == copy2[0]["ids"][16:32] and copy2[0]["answer_start"] == 16 and copy2[0]["cell"] == "n=16"


def test_recall_item_sets_plan_build_split_and_first_block(tmp_path):
    src = tmp_path / "docs.jsonl"
    src.write_text("".join(json.dumps({"id": i, "text": d}) + "\n" for i, d in enumerate(docs(50, seed=5))))
    tool = [sys.executable, str(ROOT / "scripts/build_recall_items.py")]
    run = lambda *args: subprocess.run(tool + list(args), capture_output=True, text=True, timeout=900)
    r = run("plan", "--out", str(tmp_path / "plan.json"), "--n", "100", "--n-old", "50", "--n-keys", "4", "--lengths", "2048,4096", "--budget-s", "66")
    assert r.returncode == 0, r.stderr[-1500:]
    plan = json.loads((tmp_path / "plan.json").read_text())
    assert len(plan["groups"]) >= 2 and sum(g["items"] for g in plan["groups"]) == 200
    # a small build: 3 items per cell stands in for the plan's 100 (same generator, same first items)
    small = dict(plan, cells=[dict(c, n=3, n_old=2) for c in plan["cells"]],
                 groups=[{"name": "g1", "modelled_s": 1.0, "deadline_s": 300, "items": 4, "parts": [{"cell": c["key"], "start": 0, "stop": 2} for c in plan["cells"]]},
                         {"name": "g2", "modelled_s": 1.0, "deadline_s": 300, "items": 2, "parts": [{"cell": c["key"], "start": 2, "stop": 3} for c in plan["cells"]]}])
    (tmp_path / "small.json").write_text(json.dumps(small))
    r = run("build", "--plan", str(tmp_path / "small.json"), "--out", str(tmp_path / "items"), "--tokenizer", "bytes=bytes", "--docs", str(src))
    assert r.returncode == 0, r.stderr[-1500:]
    r = run("split", "--plan", str(tmp_path / "small.json"), "--out", str(tmp_path / "items"))
    assert r.returncode == 0 and json.loads(r.stdout.strip().splitlines()[-1]) == {"groups": 2, "items_written": 6}, r.stderr[-1500:]
    g1 = torch.load(tmp_path / "items/groups/g1/bytes/multikey.pt", weights_only=False)["probes"]
    g2 = torch.load(tmp_path / "items/groups/g2/bytes/multikey.pt", weights_only=False)["probes"]
    assert [p["id"][-4:] for p in g1] == ["0000", "0001", "0000", "0001"] and [p["id"][-4:] for p in g2] == ["0002", "0002"]
    raw = tmp_path / "items/raw/bytes/multikey.pt"
    assert run("check-first-block", "--old", str(tmp_path / "items/groups/g1/bytes/multikey.pt"), "--new", str(raw)).returncode == 0
    blob = torch.load(raw, weights_only=False)
    blob["probes"][0]["ids"][5] += 1
    torch.save(blob, tmp_path / "tampered.pt")
    assert run("check-first-block", "--old", str(tmp_path / "items/groups/g1/bytes/multikey.pt"), "--new", str(tmp_path / "tampered.pt")).returncode == 4


def test_recall_items_values_from_group_outputs(tmp_path):
    from gdn_hybrid_architecture_ideas_b200.eval import recall_items as RI

    plan = RI.make_plan({"multikey_n4|2048": 6}, {"multikey_n4|2048": 2}, budget_s=70.0)
    plan["groups"] = [{"name": "g1", "modelled_s": 1.0, "deadline_s": 300, "items": 4, "parts": [{"cell": "multikey_n4|2048", "start": 0, "stop": 4}]},
                      {"name": "g2", "modelled_s": 1.0, "deadline_s": 300, "items": 2, "parts": [{"cell": "multikey_n4|2048", "start": 4, "stop": 6}]}]
    (tmp_path / "plan.json").write_text(json.dumps(plan))
    ids = [f"multikey/len=2048/n=4/{i:04d}" for i in range(6)]
    exact = [True, False, True, True, False, True]
    (tmp_path / "out").mkdir()
    (tmp_path / "out" / "g1.json").write_text(json.dumps({"items": [{"id": i, "exact": e} for i, e in zip(ids[:4], exact[:4])]}))
    tool = [sys.executable, str(ROOT / "scripts/recall_items_values.py")]
    base = ["run", "--plan", str(tmp_path / "plan.json"), "--run", "r", "--probes-dir", str(tmp_path / "out")]
    assert subprocess.run(tool + base + ["--out", str(tmp_path / "r.values.json")], capture_output=True, text=True).returncode == 3      # g2 missing
    (tmp_path / "out" / "g2.json").write_text(json.dumps({"items": [{"id": i, "exact": e} for i, e in zip(ids[4:], exact[4:])]}))
    r = subprocess.run(tool + base + ["--out", str(tmp_path / "r.values.json")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    v = json.loads((tmp_path / "r.values.json").read_text())
    assert v["cells"] == {"items|multikey_n4|2048|exact": 4 / 6} and v["family"] == "items"
    d = json.loads((tmp_path / "r.detail.json").read_text())["multikey_n4|2048"]
    assert d["first_block"] == {"n": 2, "exact": 0.5, "se": RI.binomial_se(0.5, 2)} and d["new_block"]["n"] == 4 and d["missing"] == 0
    (tmp_path / "ex.json").write_text(json.dumps(["multikey_n4:" + ids[1]]))
    r = subprocess.run(tool + base + ["--out", str(tmp_path / "x.values.json"), "--exclude-file", str(tmp_path / "ex.json")], capture_output=True, text=True)
    assert r.returncode == 0 and json.loads((tmp_path / "x.values.json").read_text())["cells"]["items|multikey_n4|2048|exact"] == 4 / 5
    (tmp_path / "bad.json").write_text(json.dumps(["multikey/len=2048/n=4/0099"]))
    assert subprocess.run(tool + base + ["--out", str(tmp_path / "y.json"), "--exclude-file", str(tmp_path / "bad.json")], capture_output=True, text=True).returncode == 3
    r = subprocess.run(tool + base + ["--out", str(tmp_path / "f.values.json"), "--first-block-only"], capture_output=True, text=True)
    assert r.returncode == 0 and json.loads((tmp_path / "f.values.json").read_text())["cells"]["items|multikey_n4|2048|exact"] == 0.5
    b = subprocess.run(tool + ["brief", "--values", str(tmp_path / "r.values.json")], capture_output=True, text=True)
    assert "0.6667" in b.stdout and "n=6" in b.stdout
