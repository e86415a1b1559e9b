"""Benchmark drivers on CPU: the all-in-one latency CSV (reference schema) and sliding-window perplexity."""
import csv
import math
import os

import torch


def test_all_in_one_csv_schema(tmp_path, monkeypatch):
    import yaml
    from ipex_llm_b200.benchmark import all_in_one
    monkeypatch.chdir(tmp_path)
    conf = {"repo_id": ["synthetic:tiny"], "warm_up": 1, "num_trials": 2, "low_bit": "sym_int8", "batch_size": 2,
            "in_out_pairs": ["16-4", "24-3"], "test_api": ["transformer_int4"]}
    with open("config.yaml", "w") as f:
        yaml.safe_dump(conf, f)
    rows = all_in_one.main(["config.yaml"])
    assert len(rows) == 2
    files = [n for n in os.listdir(".") if n.startswith("transformer_int4-results-") and n.endswith(".csv")]
    assert len(files) == 1
    with open(files[0]) as f:
        table = list(csv.reader(f))
    assert table[0][1:] == all_in_one.CSV_COLUMNS
    first = dict(zip(table[0][1:], table[1][1:]))
    assert first["input/output tokens"] == "16-4" and first["actual input/output tokens"] == "16-4"
    assert float(first["1st token avg latency (ms)"]) > 0 and float(first["2+ avg latency (ms/token)"]) > 0
    assert first["low_bit"] == "sym_int8" and first["batch_size"] == "2"


def test_perplexity_windows(tiny_llama_dir):
    from ipex_llm.transformers import AutoModelForCausalLM
    from ipex_llm_b200.benchmark.perplexity import BigDLPPL
    model = AutoModelForCausalLM.from_pretrained(tiny_llama_dir, load_in_low_bit="sym_int8")
    ppl = BigDLPPL(model=model, device="cpu")
    torch.manual_seed(0)
    ids = torch.randint(0, 32000, (96,))
    # one window over everything = the plain definition
    s, c = ppl.nll(ids)
    assert c == 95
    whole = ppl.perplexity_hf(ids, seq_len=96)
    assert abs(whole - math.exp(s / c)) < 1e-6 * whole
    # a random model on random tokens is close to uniform over the vocabulary
    assert 0.3 * 32000 < whole < 3 * 32000
    # strided windows score every token exactly once and stay in the same range
    strided = ppl.perplexity_hf(ids, seq_len=48, stride=24)
    assert 0.3 * 32000 < strided < 3 * 32000


def test_check_results_and_stress(tmp_path, monkeypatch):
    import yaml
    from ipex_llm_b200.benchmark import all_in_one, check_results, stress_test
    monkeypatch.chdir(tmp_path)
    conf = {"repo_id": ["synthetic:tiny"], "warm_up": 0, "num_trials": 1, "low_bit": "sym_int8", "batch_size": 1,
            "in_out_pairs": ["8-2"], "test_api": ["transformer_int4"]}
    with open("config.yaml", "w") as f:
        yaml.safe_dump(conf, f)
    all_in_one.main(["config.yaml"])
    assert check_results.main(["-c", "transformer_int4-results-", "-y", "config.yaml"]) == 0
    conf["in_out_pairs"].append("16-2")                 # a configured case without a row
    with open("config2.yaml", "w") as f:
        yaml.safe_dump(conf, f)
    assert check_results.main(["-c", "transformer_int4-results-", "-y", "config2.yaml"]) == 1
    rc = stress_test.main(["--repo-id", "synthetic:tiny", "--test-api", "transformer_int4", "--low-bit", "sym_int8",
                           "--in-out", "8-3", "--rounds", "3", "--max-latency-drift", "100"])
    assert rc == 0


def test_accuracy_evaluation_tools(tmp_path):
    """Likelihood scoring in lm-eval's shapes, multiple-choice accuracy by choice-letter logits, WER, LongBench
    metrics (reference dev/benchmark/{harness,ceval,whisper,LongBench})."""
    import math
    import torch
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import LlamaConfig, LlamaForCausalLM, PreTrainedTokenizerFast
    from ipex_llm import optimize_model
    from ipex_llm_b200.benchmark import evaluation as ev
    words = ["<pad>", "<s>", "</s>", "<unk>", "A", "B", "C", "D", "Answer:", "."] + [f"w{i}" for i in range(54)]
    tk = Tokenizer(models.WordLevel({w: i for i, w in enumerate(words)}, unk_token="<unk>"))
    tk.pre_tokenizer = pre_tokenizers.WhitespaceSplit()
    tok = PreTrainedTokenizerFast(tokenizer_object=tk, pad_token="<pad>", bos_token="<s>", eos_token="</s>",
                                  unk_token="<unk>")
    torch.manual_seed(0)
    cfg = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, vocab_size=64, max_position_embeddings=256, eos_token_id=2, bos_token_id=1)
    base = LlamaForCausalLM(cfg).eval()
    model = optimize_model(base, low_bit="sym_int8")
    sc = ev.LikelihoodScorer(model, tok, max_length=32)
    (lp, greedy), = sc.loglikelihood([("w1 w2 w3", "w4 w5")])
    ids = tok.encode("w1 w2 w3 w4 w5", add_special_tokens=False)
    import os
    os.environ["IPEX_LLM_LAST_LM_HEAD"] = "0"
    try:
        with torch.no_grad():
            logp = torch.log_softmax(model(torch.tensor([ids])).logits[0].float(), -1)
    finally:
        os.environ.pop("IPEX_LLM_LAST_LM_HEAD")
    want = float(logp[2, ids[3]] + logp[3, ids[4]])
    assert math.isclose(lp, want, rel_tol=1e-4) and isinstance(greedy, bool)
    best = tok.decode([int(logp[2].argmax())])
    assert sc.loglikelihood([("w1 w2 w3", best)])[0][1] is True            # the arg-max continuation is "greedy"
    long_text = " ".join(f"w{i % 50}" for i in range(80))
    (roll,) = sc.loglikelihood_rolling([(long_text,)])
    assert roll < 0 and math.isfinite(roll)
    (gen,) = sc.generate_until([("w1 w2", {"until": ["zzz"], "max_gen_toks": 4})])
    assert isinstance(gen, str)
    ev.register_with_lm_eval()                                              # a no-op without lm-eval

    mc = ev.MultipleChoiceEvaluator(model, tok)
    rows = [{"question": f"w{i} w{i + 1}", "A": "w1", "B": "w2", "C": "w3", "D": "w4", "answer": "ABCD"[i % 4]}
            for i in range(6)]
    prompt = mc.few_shot_prompt("testing", rows[:2], k=2)
    assert prompt.count("Answer:") == 2 and "A. w1" in prompt
    res = mc.eval_subject("testing", rows[2:], rows[:2], few_shot=2)
    assert 0.0 <= res["accuracy"] <= 1.0 and len(res["predictions"]) == 4 and set(res["predictions"]) <= set("ABCD")

    assert ev.word_error_rate(["the cat sat"], ["the cat sat"]) == 0.0
    assert math.isclose(ev.word_error_rate(["the cat sat on the mat"], ["the cat sit on mat"]), 2 / 6)
    assert math.isclose(ev.word_error_rate(["a b", "c d"], ["a b x", "c"]), 2 / 4)
    assert ev.truncate_middle(list(range(10)), 4) == [0, 1, 8, 9] and ev.truncate_middle([1, 2], 4) == [1, 2]
    assert ev.qa_f1_score("The Eiffel Tower", "eiffel tower") == 1.0
    assert 0 < ev.qa_f1_score("tower in paris", "eiffel tower") < 1
    assert ev.rouge_l_score("a b c d", "a c d") == 2 * (3 / 4) * 1.0 / (3 / 4 + 1.0)
    assert ev.classification_score("it is sports news", "sports", ["sports", "politics"]) == 1.0
    assert ev.retrieval_score("Paragraph 7 and maybe 3", "Paragraph 7") == 0.5
    assert ev.count_score("there are 4 or 5", "4") == 0.5
    assert ev.code_similarity_score("```\nreturn x + 1\n", "return x + 1") == 1.0
    assert ev.longbench_score("qa_f1", ["eiffel tower", "nothing"], [["Eiffel Tower", "tower"], ["paris"]]) == 50.0
