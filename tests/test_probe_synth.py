"""Probes on synthetic material: items are pure functions of their arguments, the span to write is where the context says,
distances and uniqueness hold, the stored form encodes chat pieces apart, the build script writes checked sets that the
probe scorer reads."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from gdn_hybrid_architecture_ideas_b200.data import chat_format as CF
from gdn_hybrid_architecture_ideas_b200.eval import probe_synth as PS

ROOT = Path(__file__).resolve().parent.parent
COUNT = lambda t: (len(t.encode()) + 3) // 4          # noqa: E731  a stand-in for a subword count
BYTES = lambda t: list(t.encode())                    # noqa: E731
CONTROL = PS.control_ids(256)


@pytest.mark.parametrize("length,distance,variant,form", [(8, 1024, "plain", "repeat"), (32, 4096, "near_dup", "edit"), (128, 1024, "near_dup", "repeat")])
def test_copy_items_place_the_span_at_the_distance(length, distance, variant, form):
    it = PS.copy(length, distance, variant, form, 3, COUNT)
    assert it.to_json() == PS.copy(length, distance, variant, form, 3, COUNT).to_json()
    assert it.to_json() != PS.copy(length, distance, variant, form, 3, COUNT, attempt=1).to_json()
    assert it.context.count(it.answer) == 1 and abs(COUNT(it.answer) - length) <= PS.SPAN_TOL * length
    assert PS.DIST_LO * distance <= it.meta["distance"] <= distance
    assert f"def {it.meta['target']}(value):\n{it.answer}" in it.context
    assert it.context.endswith(f"def {it.meta['target']}(value):\n" if form == "repeat" else "old_str:\n")
    floor = it.meta["floor"]
    assert floor["exact"] == 1 / floor["choices"] and floor["choices"] >= 4 and floor["exact"] <= floor["token_acc"] <= 1
    if variant == "near_dup":
        decoy, marks = it.meta["decoy"], it.meta["diff_chars"]
        assert len(marks) == PS.COPY_DIFFS[length] and decoy != it.answer and decoy in it.context
        a_lines, d_lines = it.answer.split("\n"), decoy.split("\n")
        assert len(a_lines) == len(d_lines) and sum(x != y for x, y in zip(a_lines, d_lines)) == len(marks)
        for x, y in zip(a_lines, d_lines):           # a changed line differs in one space-separated token
            assert x == y or sum(p != q for p, q in zip(x.split(" "), y.split(" "))) == 1
        word = lambda t, m: t[m:].split(" ")[0].split("\n")[0]          # noqa: E731  the token that starts at a mark
        assert it.answer[:marks[0]] == decoy[:marks[0]] and word(it.answer, marks[0]) != word(decoy, marks[0])
    else:
        assert it.meta["decoy"] is None and it.meta["diff_chars"] == []


def test_line_edit_names_the_line_of_a_definition_and_foils_share_its_context():
    for n in PS.FILE_LINES[:2]:
        for form in ("number", "sed"):
            it = PS.line_edit(n, form, 5)
            gold = it.meta["gold_line"]
            numbered = {int(row.split("\t")[0]): row.split("\t", 1)[1] for row in it.context.split("\n") if "\t" in row and row.split("\t")[0].strip().isdigit()}
            name = it.context.split("`")[1]
            assert name in numbered[gold] and sum(name in v.split("(")[0].split(" =")[0].split(":")[0] for v in numbered.values()) >= 1
            assert it.answer == (f" {gold}" if form == "number" else f"{gold}d") and gold in it.meta["definition_lines"]
            assert abs(it.meta["file_lines"] - n) <= 12 and it.meta["floor"]["definition_line"] == 1 / len(it.meta["definition_lines"])
            foils = PS.line_edit_foils(n, form, 5)
            assert foils and all(f.context == it.context and f.meta["line"] != gold and f.meta["gold_line"] == gold for f in foils)
            assert {gold + o for o in PS.FOIL_OFFSETS if 1 <= gold + o <= it.meta["file_lines"]} <= {f.meta["line"] for f in foils}
    rows = [{"question": "a", "line": 7, "gold_line": 7, "logp": -1.0}, {"question": "a", "line": 8, "gold_line": 7, "logp": -2.0},
            {"question": "b", "line": 3, "gold_line": 3, "logp": -5.0}, {"question": "b", "line": 5, "gold_line": 3, "logp": -4.0}]
    table = PS.line_choice_table(rows)
    assert table == {"questions": 2, "choice_acc": 0.5, "distance_hist": {0: 1, 2: 1}}


@pytest.mark.parametrize("kind,src,variant", [("code", "tool", "near_dup"), ("path", "assistant", "plain"), ("ident", "tool", "plain"), ("random", "assistant", "plain")])
def test_copy_span_is_a_conversation_with_the_answer_behind_a_lead_in(kind, src, variant):
    it = PS.copy_span(kind, 32, 1024, src, variant, 1, COUNT)
    assert it.to_json() == PS.copy_span(kind, 32, 1024, src, variant, 1, COUNT).to_json()
    text = it.context_text()
    assert text.count(it.answer) == 1 and text.count(f"[{it.meta['label']}]") == 2 and text.endswith("<|im_start|>assistant\n" + PS.LEADIN_COPY)
    assert not it.answer[0].isspace() and (it.answer[-1].isalnum() or it.answer[-1] == "_")
    assert 0.85 * 1024 <= it.meta["distance"] <= 1.02 * 1024
    holder = [m for m in it.conversation["messages"] if it.answer in (m.get("content") or "")]
    assert len(holder) == 1 and holder[0]["role"] == ("tool" if src == "tool" else "assistant")
    rec = PS.encode_chat_item(it, BYTES, CONTROL)
    assert all(rec["checks"].values()) and rec["ids"][rec["answer_start"]:] == BYTES(it.answer) and rec["length"] == len(rec["ids"])
    lead = BYTES(PS.LEADIN_COPY)
    assert rec["ids"][rec["answer_start"] - len(lead):rec["answer_start"]] == lead
    assert rec["ids"].count(CONTROL[CF.IM_START]) == len(it.conversation["messages"]) + 1          # the reply's header is in the context
    assert rec["floor"]["exact"] == 0.25 and abs(rec["floor"]["nats"] - 1.3862943611) < 1e-9
    if variant == "near_dup":
        assert len(rec["diff_index"]) == PS.COPY_DIFFS[32] == len(it.meta["diff_chars"])
    assert PS.copy_span(kind, 32, 1024, src, variant, 1, COUNT, leadin=None).leadin == ""
    with pytest.raises(ValueError, match="near_dup"):
        PS.copy_span("path", 8, 1024, "tool", "near_dup", 0, COUNT)


def test_edit_old_renders_one_content_four_ways():
    items = {r: PS.edit_old(3, 40, r, 2) for r in PS.RENDERS}
    first, last = items["json_num"].meta["first_line"], items["json_num"].meta["last_line"]
    assert last - first == 2 and all(it.meta["first_line"] == first and it.group == items["json_num"].group for it in items.values())
    old = items["raw_plain"].answer
    assert old.count("\n") == 2 and json.loads('"' + items["json_plain"].answer + '"') == old and items["json_num"].answer == items["json_plain"].answer
    for name, it in items.items():
        view = next(m["content"] for m in it.conversation["messages"] if m["role"] == "tool")
        plain = "\n".join(row.split("\t", 1)[1] for row in view.split("\n")) if name.endswith("_num") else view
        assert plain.count(old) == 1 and plain.split("\n")[first - 1:last] == old.split("\n")
        assert (view.split("\n")[0].split("\t")[0].strip() == "1") == name.endswith("_num")
        assert f"lines {first}-{last}" in it.conversation["messages"][-1]["content"]
        rec = PS.encode_chat_item(it, BYTES, CONTROL)
        assert all(rec["checks"].values()) and rec["ids"][rec["answer_start"] - len(BYTES(it.leadin)) - 1] == CONTROL[CF.TOOL_CALL]
        assert it.floor["exact"] == 1 / it.floor["choices"]
        if name.startswith("json"):      # lead-in + answer + suffix is the call as the chat format renders it
            call = json.loads((it.leadin + it.answer + it.suffix).strip())
            assert call == {"name": "str_replace", "arguments": {"path": it.meta["path"], "old_str": old, "new_str": "pass"}}
            assert "\n" + CF.call_json(call) + "\n" == it.leadin + it.answer + it.suffix
    with pytest.raises(ValueError, match="one of"):
        PS.edit_old(3, 40, "dec_num", 0)


@pytest.mark.parametrize("lines,kind", [(1, "code"), (3, "text"), (8, "code"), (20, "text")])
def test_transcode_directions_share_a_base_and_differ_in_form(lines, kind):
    a, b = PS.transcode("esc2raw", lines, kind, 4), PS.transcode("raw2esc", lines, kind, 4)
    raw, esc = a.answer, b.answer
    assert raw == b.meta["source"] and esc == a.meta["source"] and a.meta["base"] == b.meta["base"] and raw != esc
    assert json.loads('"' + esc + '"') == raw and raw.count("\n") == lines - 1 and "\n" not in esc
    assert any(ch in raw for ch in ('"', "\\", "\t")) and raw[0] not in '"\\' and not raw[0].isspace() and not raw[-1].isspace()
    for it, source in ((a, esc), (b, raw)):
        text = it.context_text()
        assert it.answer not in text and text.count(source) == 1
        rec = PS.encode_chat_item(it, BYTES, CONTROL)
        assert all(rec["checks"].values()) and rec["floor"]["exact"] == 0.0 and 0 < rec["floor"]["lcs_share"] <= 1
    call = json.loads((b.leadin + b.answer + b.suffix).strip())
    assert call["name"] == "write_file" and call["arguments"]["content"] == raw
    assert a.leadin == PS.LEADIN_ESC2RAW and a.reply_prefix == [] and b.reply_prefix[-1] == (CF.TOOL_CALL, True)
    assert PS.lcs(list("abcde"), list("xbdxe")) == 3
    assert PS.transcode_floor([1, 2, 3, 4], [1, 9, 3, 4, 5]) == {"exact": 0.0, "token_acc": 0.6, "lcs_share": 0.6}


def test_cell_extras_read_floors_near_duplicate_tokens_and_line_choices():
    records = [{"floor": {"exact": 0.25, "nats": 1.0}, "diff_index": [1]}, {"floor": {"exact": 0.5, "nats": 3.0}, "diff_index": [0, 2]}]
    scored = [{"ok": [True, False, True], "nats": [0.1, 2.0, 0.3]}, {"ok": [True, True, True], "nats": [0.5, 0.5, 0.5]}]
    out = PS.cell_extras(records, scored)
    assert out["floor"] == {"exact": 0.375, "nats": 2.0} and out["diff_tokens"] == 3 and abs(out["diff_acc"] - 2 / 3) < 1e-12
    assert abs(out["diff_nats"] - 1.0) < 1e-12 and abs(out["token_acc"] - 5 / 6) < 1e-12
    rows = [{"question": "q", "line": 4, "gold_line": 4, "floor": {}}, {"question": "q", "line": 5, "gold_line": 4, "floor": {}}]
    out = PS.cell_extras(rows, [{"ok": [True], "nats": [3.0]}, {"ok": [False], "nats": [1.0]}])
    assert out["line_choice"] == {"questions": 1, "choice_acc": 0.0, "distance_hist": {1: 1}}


def test_build_script_writes_checked_sets_that_the_scorer_reads(tmp_path):
    from gdn_hybrid_architecture_ideas_b200 import config as C
    from gdn_hybrid_architecture_ideas_b200.train.trainer import Trainer

    def build(out):
        r = subprocess.run([sys.executable, str(ROOT / "scripts/build_synth_probes.py"), "--out", str(out), "--tokenizer", "bytes=bytes", "--per-cell", "1",
                            "--distances", "1024", "--file-lines", "40", "--probes", "copy,line_edit_foil,copy_span,edit_old,transcode"], capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:] + r.stdout[-500:]
        return json.loads(r.stdout.strip().splitlines()[-1])

    out = tmp_path / "set"
    said = build(out)
    assert said["failed_checks"] == 0 and said["items"]["transcode"] == 2 * len(PS.TC_LINES) * len(PS.TC_KINDS) and said["items"]["edit_old"] == 4 * 6
    manifest = json.loads((out / "synth_manifest.json").read_text())
    again = tmp_path / "again"
    build(again)
    assert json.loads((again / "synth_manifest.json").read_text())["sha256"] == manifest["sha256"]            # byte-identical rebuild
    stored = torch.load(out / "bytes" / "copy_span.pt", weights_only=False)
    assert stored["vocab"] == 256 + len(CF.CONTROL_TOKENS) and all(max(p["ids"]) < stored["vocab"] for p in stored["probes"])
    model = C.tiny_full_config()
    model.vocab_size = 272
    cfg = C.TrainConfig(model=model, data=C.tiny_data_config())
    cfg.steps, cfg.log_every, cfg.metrics_jsonl, cfg.device = 1, 0, False, "cpu"
    Trainer(cfg, tmp_path / "run").fit()
    for probe in ("copy", "line_edit_foil", "transcode"):
        res = tmp_path / f"{probe}.json"
        r = subprocess.run([sys.executable, str(ROOT / "scripts/eval_probes.py"), "--checkpoint", str(tmp_path / "run"), "--set", str(out / "bytes" / f"{probe}.pt"),
                            "--device", "cpu", "--batch-size", "2", "--out", str(res)], capture_output=True, text=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        table = json.loads(res.read_text())["probes"]
        assert table and all("floor" in c and 0 <= c["token_acc"] <= 1 for c in table.values())
        if probe == "copy":
            assert any("diff_acc" in c for k, c in table.items() if "near_dup" in k) and not any("diff_acc" in c for k, c in table.items() if "plain" in k)
        if probe == "line_edit_foil":
            assert all(c["line_choice"]["questions"] == 1 and sum(c["line_choice"]["distance_hist"].values()) == 1 for c in table.values())
        if probe == "transcode":
            assert all(c["floor"]["exact"] == 0 and 0 < c["floor"]["lcs_share"] <= 1 for c in table.values())
