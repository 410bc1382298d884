"""train.py -> sharded checkpoint -> consolidated checkpoint -> eval.py (perplexity
and generation), all on CPU in child processes."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, env_extra=None):
    env = dict(os.environ)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT", "MASTER_ADDR"):
        env.pop(k, None)
    env.update({"MASTER_ADDR": "127.0.0.1", "CUDA_VISIBLE_DEVICES": ""})
    env.update(env_extra or {})
    r = subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + "\n" + r.stderr[-3000:]
    return r.stdout + r.stderr


@pytest.fixture(scope="module")
def sp_model(tmp_path_factory):
    import sentencepiece as spm
    d = tmp_path_factory.mktemp("sp")
    corpus = d / "corpus.txt"
    words = ["alpha", "beta", "gamma", "delta", "omega", "shark", "ocean", "long", "context", "model"]
    with open(corpus, "w") as f:
        for i in range(400):
            f.write(" ".join(words[(i * 7 + j * 3) % len(words)] for j in range(12)) + ".\n")
    prefix = str(d / "tok")
    spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=prefix, vocab_size=64, model_type="bpe",
                                   bos_id=1, eos_id=2, pad_id=0, unk_id=3)
    return prefix + ".model", words


def test_train_consolidate_eval_roundtrip(tmp_path, sp_model):
    tok_path, words = sp_model
    data = tmp_path / "train.jsonl"
    with open(data, "w") as f:
        for i in range(8):
            f.write(json.dumps({"text": " ".join(words[(i + j) % len(words)] for j in range(400))}) + "\n")
    run_dir, cons_dir, dump = tmp_path / "run", tmp_path / "cons", tmp_path / "eval"
    out = _run(["train.py", "--model", "mega_tiny", "--vocab_size", "64", "--steps", "3", "--seq_len", "128",
                "--batch_size", "2", "--dtype", "fp32", "--warmup", "1", "--lr", "0.01", "--dump_dir", str(run_dir),
                "--save_every", "2", "--consolidate_to", str(cons_dir), "--data_path", str(data),
                "--tokenizer_path", tok_path])
    assert "step 3 loss" in out and "Finished training" in out
    assert (run_dir / "model.ckpt.00000.pth").exists() and (run_dir / "metrics.jsonl").exists()
    assert (cons_dir / "consolidated.pth").exists() and (cons_dir / "consolidate_config.json").exists()
    # resume continues from the saved step
    out = _run(["train.py", "--model", "mega_tiny", "--vocab_size", "64", "--steps", "4", "--seq_len", "128",
                "--batch_size", "2", "--dtype", "fp32", "--warmup", "1", "--dump_dir", str(run_dir),
                "--resume", "true"])
    assert "resumed from step 3" in out and "step 4 loss" in out

    ppl_file = tmp_path / "valid.jsonl"
    with open(ppl_file, "w") as f:
        for i in range(3):
            f.write(json.dumps({"text": " ".join(words[(2 * i + j) % len(words)] for j in range(150))}) + "\n")
    prompts = tmp_path / "prompts.jsonl"
    with open(prompts, "w") as f:
        f.write(json.dumps({"text": "alpha beta gamma"}) + "\n")
        f.write(json.dumps({"text": "ocean shark"}) + "\n")
    out = _run(["eval.py", "--checkpoint_dir", str(cons_dir), "--dump_dir", str(dump), "--tokenizer_path", tok_path,
                "--dtype", "fp32", "--ppl_files_str", str(ppl_file), "--prompt_path", str(prompts),
                "--gen_seq_len", "8", "--batch_size", "2"])
    assert "PPL on" in out and "Finished all evaluations" in out
    assert "Missing keys when reloading" not in out and "Unexpected keys when reloading" not in out
    gens = [json.loads(l) for l in open(dump / "generations" / "0.jsonl")]
    assert [g["prompt"] for g in gens] == ["alpha beta gamma", "ocean shark"]
