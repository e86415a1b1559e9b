"""Accuracy evaluation tools: likelihood scoring for lm-eval style tasks, multiple-choice exams, word error rate,
long-context answer metrics.

The reference keeps these as scripts under python/llm/dev/benchmark/: ``harness/ipexllm.py`` (an lm-eval ``LM`` that
loads the model with ``load_in_low_bit``), ``ceval/`` (few-shot multiple-choice exam evaluators that compare the
logits of the choice letters), ``whisper/`` (word error rate on LibriSpeech) and ``LongBench/`` (``pred.py`` with
middle truncation of long prompts, ``metrics.py``).  Here they are one importable module on the package's models:

* ``LikelihoodScorer``: ``loglikelihood`` / ``loglikelihood_rolling`` / ``generate_until`` with the request and result
  shapes lm-eval uses, so an lm-eval task can be driven by it (``register_with_lm_eval`` wraps it in an ``LM`` when
  that package is installed);
* ``MultipleChoiceEvaluator``: few-shot prompt assembly and accuracy by the logits of the choice letters;
* ``word_error_rate``;
* ``truncate_middle`` and the LongBench answer metrics (``qa_f1_score``, ``rouge_l_score``, ``classification_score``,
  ``retrieval_score``, ``count_score``, ``code_similarity_score``).
"""
from __future__ import annotations

import re
import string
from collections import Counter
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch


# ------------------------------------------------------------------------------------------------
# likelihood scoring (lm-eval request shapes)
# ------------------------------------------------------------------------------------------------
class LikelihoodScorer:
    def __init__(self, model, tokenizer, max_length: int = 2048, batch_size: int = 1):
        self.model, self.tokenizer, self.max_length, self.batch_size = model, tokenizer, max_length, batch_size

    @classmethod
    def from_pretrained(cls, path: str, load_in_low_bit: str = "sym_int4", device: str = None, **kw):
        from transformers import AutoTokenizer
        from ..transformers import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(path, load_in_low_bit=load_in_low_bit, **kw).eval()
        device = device or ("cuda" if torch.cuda.is_available() else "cpu")
        return cls(model.to(device), AutoTokenizer.from_pretrained(path))

    @property
    def device(self):
        return next(self.model.parameters()).device

    def _encode(self, text: str) -> List[int]:
        return list(self.tokenizer.encode(text, add_special_tokens=False))

    def _full_logits(self, ids: List[int]) -> torch.Tensor:
        """Logits at every position (the last-token shortcut of the lm_head is switched off for the call)."""
        import os
        prev = os.environ.get("IPEX_LLM_LAST_LM_HEAD")
        os.environ["IPEX_LLM_LAST_LM_HEAD"] = "0"
        try:
            with torch.no_grad():
                out = self.model(torch.tensor([ids], device=self.device)).logits[0].float()
        finally:
            if prev is None:
                os.environ.pop("IPEX_LLM_LAST_LM_HEAD", None)
            else:
                os.environ["IPEX_LLM_LAST_LM_HEAD"] = prev
        return out

    def _score(self, ctx: List[int], cont: List[int]) -> Tuple[float, bool]:
        ids = (ctx + cont)[-(self.max_length + 1):]
        n = min(len(cont), len(ids) - 1)
        logp = torch.log_softmax(self._full_logits(ids[:-1]), dim=-1)[-n:]
        tgt = torch.tensor(ids[-n:], device=logp.device)
        greedy = bool((logp.argmax(-1) == tgt).all())
        return float(logp.gather(1, tgt.unsqueeze(1)).sum()), greedy

    def loglikelihood(self, requests: Iterable[Tuple[str, str]]) -> List[Tuple[float, bool]]:
        """``[(context, continuation)] -> [(log p(continuation | context), continuation is the greedy choice)]``."""
        out = []
        bos = self.tokenizer.bos_token_id
        for context, continuation in requests:
            ctx = self._encode(context) if context else ([bos] if bos is not None else [])
            if not ctx:
                ctx = [self.tokenizer.eos_token_id or 0]
            out.append(self._score(ctx, self._encode(continuation)))
        return out

    def loglikelihood_rolling(self, requests: Iterable[Tuple[str]]) -> List[float]:
        """Total log-likelihood of each text, in windows of ``max_length`` tokens."""
        res = []
        start = self.tokenizer.bos_token_id
        if start is None:
            start = self.tokenizer.eos_token_id or 0
        for (text,) in requests:
            toks = self._encode(text)
            total, pos = 0.0, 0
            prefix = [start]
            while pos < len(toks):
                window = toks[pos:pos + self.max_length]
                total += self._score(prefix, window)[0]
                prefix = [window[-1]]
                pos += len(window)
            res.append(total)
        return res

    def generate_until(self, requests: Iterable[Tuple[str, dict]]) -> List[str]:
        res = []
        for context, args in requests:
            until = args.get("until") or []
            until = [until] if isinstance(until, str) else list(until)
            ids = torch.tensor([self._encode(context)[-self.max_length:]], device=self.device)
            with torch.no_grad():
                out = self.model.generate(ids, max_new_tokens=int(args.get("max_gen_toks", 256)), do_sample=False)
            text = self.tokenizer.decode(out[0, ids.shape[1]:], skip_special_tokens=True)
            for stop in until:
                if stop and stop in text:
                    text = text[: text.index(stop)]
            res.append(text)
        return res


def register_with_lm_eval(name: str = "ipex-llm"):
    """Expose ``LikelihoodScorer`` as an lm-eval model named ``name``; returns the class, or None without lm-eval."""
    try:
        from lm_eval.api.model import LM
        from lm_eval.api.registry import register_model
    except Exception:  # noqa: BLE001
        return None

    @register_model(name)
    class IPEXLLM(LM):
        def __init__(self, pretrained: str, load_in_low_bit: str = "sym_int4", max_length: int = 2048, **kw):
            super().__init__()
            self.scorer = LikelihoodScorer.from_pretrained(pretrained, load_in_low_bit)
            self.scorer.max_length = int(max_length)

        def loglikelihood(self, requests):
            return self.scorer.loglikelihood([r.args for r in requests])

        def loglikelihood_rolling(self, requests):
            return self.scorer.loglikelihood_rolling([r.args for r in requests])

        def generate_until(self, requests):
            return self.scorer.generate_until([r.args for r in requests])
    return IPEXLLM


# ------------------------------------------------------------------------------------------------
# multiple-choice exams (C-Eval / MMLU style rows: question, A, B, C, D, answer)
# ------------------------------------------------------------------------------------------------
class MultipleChoiceEvaluator:
    def __init__(self, model, tokenizer, choices: Sequence[str] = ("A", "B", "C", "D"), max_length: int = 2048):
        self.model, self.tokenizer, self.choices, self.max_length = model, tokenizer, list(choices), max_length
        self.choice_ids = [tokenizer.encode(c, add_special_tokens=False)[-1] for c in self.choices]

    def format_example(self, row: Dict[str, str], include_answer: bool = True) -> str:
        text = row["question"]
        for c in self.choices:
            text += f"\n{c}. {row[c]}"
        text += "\nAnswer:"
        if include_answer:
            text += f" {row['answer']}\n\n"
        return text

    def few_shot_prompt(self, subject: str, dev_rows: Sequence[Dict[str, str]], k: int = 5) -> str:
        head = f"The following are multiple-choice questions about {subject}. Choose the correct answer.\n\n"
        return head + "".join(self.format_example(r, True) for r in list(dev_rows)[:k])

    def predict(self, prompt: str) -> str:
        ids = self.tokenizer.encode(prompt)[-self.max_length:]
        dev = next(self.model.parameters()).device
        with torch.no_grad():
            logits = self.model(torch.tensor([ids], device=dev)).logits[0, -1].float()
        return self.choices[int(logits[self.choice_ids].argmax())]

    def eval_subject(self, subject: str, test_rows: Sequence[Dict[str, str]], dev_rows: Sequence[Dict[str, str]] = (),
                     few_shot: int = 5) -> Dict[str, object]:
        head = self.few_shot_prompt(subject, dev_rows, few_shot) if dev_rows and few_shot else ""
        preds = [self.predict(head + self.format_example(r, False)) for r in test_rows]
        correct = sum(p == r["answer"] for p, r in zip(preds, test_rows))
        return {"subject": subject, "accuracy": correct / max(len(test_rows), 1), "predictions": preds}


# ------------------------------------------------------------------------------------------------
# speech: word error rate
# ------------------------------------------------------------------------------------------------
def _words(text: str) -> List[str]:
    text = text.lower().translate(str.maketrans("", "", string.punctuation))
    return text.split()


def word_error_rate(references: Sequence[str], hypotheses: Sequence[str]) -> float:
    """(substitutions + deletions + insertions) / reference words, over the whole set."""
    errors = total = 0
    for ref, hyp in zip(references, hypotheses):
        r, h = _words(ref), _words(hyp)
        prev = list(range(len(h) + 1))
        for i, rw in enumerate(r, 1):
            cur = [i] + [0] * len(h)
            for j, hw in enumerate(h, 1):
                cur[j] = min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (rw != hw))
            prev = cur
        errors += prev[-1]
        total += len(r)
    return errors / max(total, 1)


# ------------------------------------------------------------------------------------------------
# long context: prompt truncation and answer metrics
# ------------------------------------------------------------------------------------------------
def truncate_middle(token_ids: Sequence[int], max_length: int) -> List[int]:
    """Keep the first and the last ``max_length / 2`` tokens: instructions sit at both ends of a long-context prompt."""
    ids = list(token_ids)
    if len(ids) <= max_length:
        return ids
    half = max_length // 2
    return ids[:half] + ids[len(ids) - (max_length - half):]


def _normalize_answer(s: str) -> str:
    s = s.lower().translate(str.maketrans("", "", string.punctuation))
    s = re.sub(r"\b(a|an|the)\b", " ", s)
    return " ".join(s.split())


def _f1(pred_tokens: List[str], truth_tokens: List[str]) -> float:
    common = Counter(pred_tokens) & Counter(truth_tokens)
    same = sum(common.values())
    if same == 0:
        return 0.0
    p, r = same / len(pred_tokens), same / len(truth_tokens)
    return 2 * p * r / (p + r)


def qa_f1_score(prediction: str, ground_truth: str) -> float:
    return _f1(_normalize_answer(prediction).split(), _normalize_answer(ground_truth).split())


def _lcs(a: List[str], b: List[str]) -> int:
    prev = [0] * (len(b) + 1)
    for x in a:
        cur = [0]
        for j, y in enumerate(b, 1):
            cur.append(prev[j - 1] + 1 if x == y else max(prev[j], cur[j - 1]))
        prev = cur
    return prev[-1]


def rouge_l_score(prediction: str, ground_truth: str) -> float:
    p, t = prediction.split(), ground_truth.split()
    if not p or not t:
        return 0.0
    l = _lcs(p, t)
    if l == 0:
        return 0.0
    prec, rec = l / len(p), l / len(t)
    return 2 * prec * rec / (prec + rec)


def classification_score(prediction: str, ground_truth: str, all_classes: Sequence[str]) -> float:
    hits = [c for c in all_classes if c in prediction]
    hits = [c for c in hits if not (c != ground_truth and c in ground_truth)]
    return 1.0 / len(hits) if ground_truth in hits else 0.0


def retrieval_score(prediction: str, ground_truth: str) -> float:
    """The answer names a paragraph number ("Paragraph 7"): the fraction of numbers in the prediction that equal it."""
    m = re.findall(r"\d+", ground_truth)
    nums = re.findall(r"\d+", prediction)
    if not m or not nums:
        return 0.0
    return sum(n == m[0] for n in nums) / len(nums)


def count_score(prediction: str, ground_truth: str) -> float:
    nums = re.findall(r"\d+", prediction)
    return sum(n == str(ground_truth) for n in nums) / len(nums) if nums else 0.0


def code_similarity_score(prediction: str, ground_truth: str) -> float:
    """Edit similarity of the first code line of the prediction with the expected line."""
    line = next((ln for ln in prediction.lstrip("\n").split("\n") if ln.strip() and "`" not in ln
                 and not ln.lstrip().startswith("#")), "")
    a, b = line.strip(), ground_truth.strip()
    if not a and not b:
        return 1.0
    prev = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        cur = [i] + [0] * len(b)
        for j, cb in enumerate(b, 1):
            cur[j] = min(prev[j] + 1, cur[j - 1] + 1, prev[j - 1] + (ca != cb))
        prev = cur
    return 1.0 - prev[-1] / max(len(a), len(b))


LONGBENCH_METRICS = {"qa_f1": qa_f1_score, "rouge_l": rouge_l_score, "classification": classification_score,
                     "retrieval": retrieval_score, "count": count_score, "code_sim": code_similarity_score}


def longbench_score(metric: str, predictions: Sequence[str], answers: Sequence[Sequence[str]],
                    all_classes: Optional[Sequence[str]] = None) -> float:
    """Mean over samples of the best score against any of the sample's reference answers, in percent."""
    fn = LONGBENCH_METRICS[metric]
    total = 0.0
    for pred, refs in zip(predictions, answers):
        best = 0.0
        for ref in refs:
            best = max(best, fn(pred, ref, all_classes) if metric == "classification" else fn(pred, ref))
        total += best
    return round(100.0 * total / max(len(predictions), 1), 2)
