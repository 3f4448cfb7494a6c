"""Evaluation / data scripts on CPU with a tiny random model and a toy tokenizer-free corpus."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "scripts"))


def test_longbench_metrics():
    import longbench_metrics as m
    assert m.qa_f1_score("The cat sat.", "a cat sat") == 1.0
    assert 0 < m.rouge_score("the quick brown fox", "the brown fox jumps") < 1
    assert m.retrieval_score("It is Paragraph 7 or 3", "Paragraph 7") == 0.5
    assert m.count_score("there are 4, maybe 4", "4") == 1.0
    assert m.classification_score("class: sports", "sports", all_classes=["sports", "politics"]) == 1.0
    assert m.scorer("trec", ["sports\njunk politics"], [["sports"]], ["sports", "politics"]) == 100.0
    assert m.code_sim_score("\nreturn x + 1\n", "return x + 1") == 1.0


def test_ruler_string_match_and_file_lookup(tmp_path):
    import eval_ruler as r
    assert r.string_match_all(["the key is 1234 and 99"], [["1234", "77"]]) == 50.0
    f = tmp_path / "4096" / "niah_single_1"
    f.mkdir(parents=True)
    (f / "validation.jsonl").write_text(json.dumps({"input": "x", "outputs": ["y"]}) + "\n")
    assert r.find_file(tmp_path, "niah_single_1", 4096) is not None
    assert r.find_file(tmp_path, "niah_single_1", 8192) is None


def test_greedy_decode_and_token_nll_on_a_tiny_model():
    import eval_common as c
    from ttcd_b200.models import TransformerConfig, TransformerForCausalLM
    torch.manual_seed(0)
    model = TransformerForCausalLM(TransformerConfig(hidden_size=32, num_hidden_layers=2, num_heads=4, num_kv_heads=2,
                                                     intermediate_size=64, vocab_size=64, window_size=16, fuse_cross_entropy=False,
                                                     fuse_linear_cross_entropy=False, max_position_embeddings=128)).eval()
    ids = torch.randint(0, 64, (1, 20))
    out = c.greedy_decode(model, ids, 5)
    full = model.generate(ids, max_new_tokens=5)
    assert out == full[0, 20:].tolist()                      # same tokens as the model's own generate
    nll = c.token_nll(model, ids, chunk=7)
    ref = torch.nn.functional.cross_entropy(model(input_ids=ids).logits[0, :-1].float(), ids[0, 1:], reduction="none")
    torch.testing.assert_close(nll[0], ref, rtol=1e-5, atol=1e-5)


def test_prepare_books_and_summarize_logs(tmp_path):
    src = tmp_path / "corpus"
    src.mkdir()
    for i in range(5):
        (src / f"doc{i}.txt").write_text("word " * (50 * (i + 1)))
    out = tmp_path / "books"
    res = subprocess.run([sys.executable, str(ROOT / "scripts" / "prepare_books.py"), "--input", str(src), "--output", str(out),
                          "--docs_per_shard", "2", "--min_chars", "300"], capture_output=True, text=True, check=True)
    info = json.loads(res.stdout.strip().splitlines()[-1])
    assert info["documents"] == 4 and info["dropped_short"] == 1 and info["shards"] == 2
    import pyarrow.parquet as pq
    assert len(pq.read_table(out / "shard_00000.parquet")["text"]) == 2
    log = tmp_path / "train.log"
    log.write_text("\n".join(f"step: {s}  loss: 2.5  tps: {1000 + s:,}  tflops: 1.0  mfu: 40.00%" for s in range(1, 8)))
    res = subprocess.run([sys.executable, str(ROOT / "scripts" / "summarize_step_metrics.py"), str(log), "--skip", "2"],
                         capture_output=True, text=True, check=True)
    row = json.loads(res.stdout.strip())
    assert row["steps"] == 5 and row["tps_mean"] == 1005.0 and row["mfu_mean"] == 40.0


class _WordTokenizer:
    """Whitespace tokenizer with the call shape the scripts use."""
    truncation_side = "right"

    def __call__(self, text, add_special_tokens=False, return_attention_mask=False, truncation=False, max_length=None,
                 return_tensors=None):
        from types import SimpleNamespace

        def enc(t):
            ids = [hash(w) % 251 for w in t.split()]
            if truncation and max_length is not None and len(ids) > max_length:
                ids = ids[-max_length:] if self.truncation_side == "left" else ids[:max_length]
            return ids
        if isinstance(text, list):
            return {"input_ids": [enc(t) for t in text]}
        return SimpleNamespace(input_ids=enc(text))


def test_ruler_data_generator_fits_the_context_and_hides_the_answers():
    import random

    import gen_ruler_data as g
    tok = _WordTokenizer()
    for task in g.ALL_TASKS:
        family = "niah" if task in g.NIAH_TASKS else task
        d = g.make_sample(task, tok, 1024, random.Random(task))
        assert d["length"] <= 1024 - g.TOKENS_TO_GENERATE[family] + len(d["answer_prefix"].split()), task
        assert d["length"] > 600, (task, d["length"])                 # the prompt is grown to (nearly) fill the context
        assert d["outputs"] and all(o in d["input"] for o in d["outputs"]), task
    multi = g.make_sample("niah_multivalue", tok, 512, random.Random(1))
    assert len(multi["outputs"]) == 4
    vt = g.make_sample("vt", tok, 512, random.Random(2))
    assert len(vt["outputs"]) == 5
    order = [vt["input"].index(f"VAR {v} =") for v in vt["outputs"]]
    assert order == sorted(order)                                      # the chain appears in assignment order


def test_final_block_eval_manifest_and_merges(tmp_path):
    import numpy as np

    import eval_final_block_doc_ppl as ffb
    import merge_eval_results as mg
    from ttcd_b200.models import TransformerConfig, TransformerForCausalLM
    import pyarrow as pa
    import pyarrow.parquet as pq
    texts = [" ".join(f"w{(i * 7 + j) % 97}" for j in range(n)) for i, n in enumerate([40, 120, 300, 90, 260])]
    pq.write_table(pa.table({"text": texts}), tmp_path / "a.parquet")
    docs, stats = ffb.select_documents(_WordTokenizer(), [str(tmp_path / "a.parquet")], seq_len=200, token_budget=10 ** 6,
                                       min_doc_tokens=100)
    assert [len(d) for d in docs] == [120, 200, 200] and stats["eligible_docs"] == 3 and stats["sampled_docs"] == 5
    ffb.save_manifest(str(tmp_path / "m.npz"), docs, stats)
    docs2, stats2 = ffb.load_manifest(str(tmp_path / "m.npz"))
    assert stats2 == stats and all(np.array_equal(a, b) for a, b in zip(docs, docs2))

    torch.manual_seed(0)
    model = TransformerForCausalLM(TransformerConfig(hidden_size=32, num_hidden_layers=1, num_heads=4, num_kv_heads=2,
                                                     intermediate_size=64, vocab_size=256, window_size=64, fuse_cross_entropy=False,
                                                     fuse_linear_cross_entropy=False, max_position_embeddings=256)).eval()
    rows = ffb.final_block_curve(model, docs, [16, 100, 150], block=32, batch_size=2, device="cpu")
    assert [r["num_sequences"] for r in rows] == [3, 2, 2] and rows[0]["total_pred_tokens"] == 96
    ids = torch.from_numpy(docs[0][-48:].astype("int64"))[None]
    want = torch.nn.functional.cross_entropy(model(input_ids=ids).logits[0, 15:-1].float(), ids[0, 16:], reduction="sum")
    one = ffb.final_block_curve(model, docs[:1], [16], block=32, batch_size=1, device="cpu")[0]
    assert abs(one["avg_nll"] * 32 - float(want)) < 1e-3

    meta = {"seq_len": 200, "final_block_size": 32, "context_lens": [16, 100, 150], "selected_total_tokens": 520,
            "min_doc_tokens": 100, "num_documents": 3}
    for name in ("a", "b"):
        (tmp_path / name).mkdir()
        ffb.write_outputs(tmp_path / name, meta, stats, {name: rows})
    merged = mg.merge_final_block([str(tmp_path / "a"), str(tmp_path / "b" / "fixed_final_block_doc_ppl.json")], str(tmp_path / "ab"))
    assert list(merged["results"]) == ["a", "b"]
    assert (tmp_path / "ab" / "fixed_final_block_doc_ppl.csv").read_text().splitlines()[0] == "context_len,a,b"

    for seed, n, v in ((1, 2, 1.0), (2, 6, 2.0)):
        (tmp_path / f"s{seed}.json").write_text(json.dumps({"seq_len": 5, "num_samples": n, "nll_per_position": [v] * 4}))
    out = mg.merge_offset_shards([str(tmp_path / "s1.json"), str(tmp_path / "s2.json")], str(tmp_path / "s.json"))
    assert out["num_samples"] == 8 and abs(out["nll"] - 1.75) < 1e-12

    import report_results as rr
    text, by_task = rr.niah_tables({"m": {"4096": {"niah_single_1": {"accuracy": 80.0}, "average": 80.0}}})
    assert "niah_single_1" in text and by_task["average"]["m"][4096] == 80.0
    rr.main(["final-block", "--input", str(tmp_path / "ab" / "fixed_final_block_doc_ppl.json")])
    rr.main(["token-ppl", "--inputs", f"x={tmp_path / 's.json'}"])
    # figures: matplotlib where it is installed, else the built-in SVG writer (same name, .svg)
    rr.main(["final-block", "--input", str(tmp_path / "ab" / "fixed_final_block_doc_ppl.json"), "--fig", str(tmp_path / "fig" / "ffb.png")])
    written = list((tmp_path / "fig").glob("ffb.*"))
    assert len(written) == 1
    if written[0].suffix == ".svg":
        svg = written[0].read_text()
        assert svg.startswith("<svg") and svg.count("<polyline") == 2 and "perplexity of the final block" in svg
    ax = rr._SvgAxes()
    ax.plot([1024, 2048, 4096], [3.0, 2.5, 2.25], marker="o", label="m")
    ax.set_xscale("log", base=2)
    ax.save(tmp_path / "fig" / "direct.svg")
    assert (tmp_path / "fig" / "direct.svg").read_text().count("<circle") == 3


def test_verify_configs_reports_every_config():
    import verify_configs
    assert verify_configs.main(["--build"]) == 0


def test_checkpoint_bench_runs_both_attention_implementations(tmp_path):
    """benchmarks/bench_checkpoint.py: timing + predictions with the fused and the two-call dual attention agree."""
    sys.path.insert(0, str(ROOT / "benchmarks"))
    import bench_checkpoint as bc
    from ttcd_b200 import ops
    from ttcd_b200.models import IPTTCDv9Config, IPTTCDForCausalLM

    class Tok:
        eos_token_id = None

        def __call__(self, text, return_tensors=None, add_special_tokens=False):
            from types import SimpleNamespace
            return SimpleNamespace(input_ids=torch.tensor([[(ord(c) * 7) % 61 for c in text]]))

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(i) for i in ids)

    data = tmp_path / "validation.jsonl"
    data.write_text("\n".join(json.dumps({"input": "abcdefgh" * (4 + i), "answer_prefix": " ans", "outputs": ["1"]}) for i in range(3)))
    torch.manual_seed(0)
    model = IPTTCDForCausalLM(IPTTCDv9Config(hidden_size=32, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                                             intermediate_size=64, vocab_size=64, window_size=24, window_size_student=8,
                                             ttt_mode=True, ttt_chunk=8, ttt_layers=[1], fuse_cross_entropy=False,
                                             fuse_linear_cross_entropy=False, max_position_embeddings=256)).eval()
    prompts, refs = bc.load_prompts(str(data), 2)
    assert len(prompts) == 3 and prompts[0].endswith(" ans")
    dev = torch.device("cpu")
    a = bc.run(model, Tok(), prompts, refs, 4, dev, "fused")
    ops.set_dual_attention_impl("two_pass")
    try:
        b = bc.run(model, Tok(), prompts, refs, 4, dev, "two_pass")
    finally:
        ops.set_dual_attention_impl("fused")
    assert len(a["predictions"]) == 2 and a["predictions"] == b["predictions"]
    assert a["median_prefill_ms"] > 0 and "decode_ms_per_token" in a


def test_ab_harness_reports_agreement_of_two_arms(tmp_path, monkeypatch):
    """scripts/eval_ab.py on a tiny random model: the task suite (prediction identity), NLL per arm and the KL pass
    between the two dual-attention implementations, written to one report."""
    import eval_ab as ab
    from ttcd_b200.models import IPTTCDv9Config, IPTTCDForCausalLM

    class Tok:
        eos_token_id = None

        def __call__(self, text, return_tensors=None, add_special_tokens=False):
            from types import SimpleNamespace
            return SimpleNamespace(input_ids=torch.tensor([[(ord(c) * 7) % 61 for c in text]]))

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(i) for i in ids)

    torch.manual_seed(0)
    model = IPTTCDForCausalLM(IPTTCDv9Config(hidden_size=32, num_hidden_layers=2, num_heads=4, num_kv_heads=2, head_dim=8,
                                             intermediate_size=64, vocab_size=64, window_size=24, window_size_student=8,
                                             ttt_mode=True, ttt_chunk=8, ttt_layers=[1], fuse_cross_entropy=False,
                                             fuse_linear_cross_entropy=False, max_position_embeddings=256)).eval()
    monkeypatch.setattr(ab, "load_model", lambda args: model)
    monkeypatch.setattr(ab, "load_tokenizer", lambda path: Tok())
    d = tmp_path / "ctx64" / "niah_single_1"
    d.mkdir(parents=True)
    (d / "validation.jsonl").write_text("\n".join(
        json.dumps({"input": "abcdefgh" * (4 + i), "answer_prefix": " ans", "outputs": ["1"]}) for i in range(3)))
    out = tmp_path / "ab.json"
    rep = ab.main(["--tokenizer", "none", "--device", "cpu", "--data_dir", str(tmp_path), "--tasks", "niah_single_1",
                   "--ctx_lens", "64", "--max_samples", "2", "--max_new_tokens", "4", "--seq_len", "48", "--ppl_docs", "3",
                   "--kl_docs", "2", "--output", str(out)])
    saved = json.loads(out.read_text())
    assert saved["arm_a"] == {"attn": "two_pass", "decode": "eager"} and saved["arm_b"] == {"attn": "fused", "decode": "graph"}
    assert saved["identical_predictions"] == [2, 2] and saved["tasks"]["niah_single_1@64"]["n"] == 2
    dist = saved["distribution"]
    assert dist["docs"] == 3 and dist["kl_tokens"] == 2 * 48 and dist["kl_max"] < 1e-6 and dist["top1_flip_rate"] == 0.0
    assert abs(dist["nll_diff"]) < 1e-5 and rep["arms_agree"] is True
    with pytest.raises(SystemExit):
        ab.parse_arm("attn=flash")
