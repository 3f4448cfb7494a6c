"""Evaluation / data scripts on CPU with a tiny random model and a toy tokenizer-free corpus."""
import json
import subprocess
import sys
from pathlib import Path

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
