"""LongEval long-context retrieval tasks ("lines" and "topics") run through this framework's generation.

A test case is one JSON line.  "lines": a long record of `line <name>: REGISTER_CONTENT is <number>` entries followed by
the question for one of them; the answer is the last integer of the model's output and the score is exact-match
accuracy.  "topics": a conversation over several topics followed by "what was the first topic"; outputs are written
for inspection (the reference does not score them either).  Files follow the LongEval layout
`<test_dir>/lines/testcases/<n>_lines.jsonl` and `<test_dir>/topics/testcases/<n>_topics.jsonl`; responses go to
`evaluation/<task>/predictions/<model name>/<n>_response.txt` with the summary line format
`Label: ..., Predict: ..., Parsed: ..., prompt length: ...` and a final `Accuracy: ...` line.

Role of the reference's savanna/inference/longeval.py:14-368 (task loops :274-338, per-sample tests :107-271).  That
file also drives third-party chat models downloaded from a hub; here the evaluated model is a checkpoint of this
framework (`inference/load.py`), and `make_lines_testcases` / `make_topics_testcases` write the test files locally, so
the evaluation runs without network access.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import re
from typing import Dict, Iterable, List, Optional, Tuple

LINES_SIZES = (200, 300, 400, 500, 600, 680)
TOPICS_SIZES = (5, 10, 15, 20, 25)

_WORDS = ("amber", "birch", "cedar", "delta", "ember", "fjord", "grove", "heron", "inlet", "jade", "kelp", "lotus",
          "maple", "north", "opal", "pearl", "quartz", "reed", "slate", "tidal", "umber", "vale", "wren", "yarrow")


# ------------------------------------------------------------------------------------------------ test-case files
def make_lines_testcases(num_lines: int, num_cases: int, seed: int = 0) -> List[Dict]:
    """Line-retrieval cases: `num_lines` register lines with distinct two-word names and random 5-digit values."""
    rng = random.Random(seed * 7919 + num_lines)
    cases = []
    for _ in range(num_cases):
        names = set()
        while len(names) < num_lines:
            names.add(f"{rng.choice(_WORDS)}-{rng.choice(_WORDS)}-{rng.randrange(10 ** 4)}")
        names = list(names)
        values = [rng.randrange(10 ** 4, 10 ** 5) for _ in names]
        body = "\n".join(f"line {n}: REGISTER_CONTENT is <{v}>" for n, v in zip(names, values))
        pick = rng.randrange(num_lines)
        prompt = ("Below is a record of lines I want you to remember. Each line begins with 'line <line index>' and "
                  "contains a '<REGISTER_CONTENT>' at the end of the line as a numerical value. For each line index, "
                  f"memorize its corresponding <REGISTER_CONTENT>.\n{body}\nNow the record is over. Tell me what is the "
                  f"<REGISTER_CONTENT> in line {names[pick]}? I need the number.")
        cases.append({"random_idx": [names[pick], pick], "name": f"{num_lines}_lines", "prompt": prompt,
                      "correct_line": f"line {names[pick]}: REGISTER_CONTENT is <{values[pick]}>",
                      "expected_number": values[pick], "num_lines": num_lines})
    return cases


def make_topics_testcases(num_topics: int, num_cases: int, seed: int = 0, turns_per_topic: int = 4) -> List[Dict]:
    """Topic-retrieval cases: a conversation that moves through `num_topics` topics; the label is the first one."""
    rng = random.Random(seed * 104729 + num_topics)
    cases = []
    for _ in range(num_cases):
        topics = [f"the {rng.choice(_WORDS)} {rng.choice(_WORDS)} project {rng.randrange(1000)}" for _ in range(num_topics)]
        parts = []
        for t in topics:
            parts.append(f"USER: I would like to discuss the topic of {t}.")
            for k in range(turns_per_topic):
                parts.append(f"ASSISTANT: Here is point {k + 1} about {t}: it involves {rng.choice(_WORDS)} and {rng.choice(_WORDS)}.")
                parts.append("USER: Tell me more.")
        prompt = ("Below is a record of our previous conversation on {n} different topics. You are the ASSISTANT, and I am "
                  "the USER. At the beginning of each topic, the USER will say 'I would like to discuss the topic of "
                  "<TOPIC>'. Memorize each <TOPIC>. At the end of the record, I will ask you to retrieve the first topic.\n"
                  "{body}\nNow the record is over. What is the first topic we discussed? Only give me the topic name."
                  ).format(n=num_topics, body="\n".join(parts))
        cases.append({"topics": topics, "prompt": prompt, "num_topics": num_topics})
    return cases


def write_testcases(test_dir: str, task: str, sizes: Optional[Iterable[int]] = None, num_cases: int = 50, seed: int = 0) -> List[str]:
    sizes = tuple(sizes) if sizes else (LINES_SIZES if task == "lines" else TOPICS_SIZES)
    out = []
    for n in sizes:
        path = testcase_path(test_dir, task, n)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        cases = make_lines_testcases(n, num_cases, seed) if task == "lines" else make_topics_testcases(n, num_cases, seed)
        with open(path, "w") as fh:
            for c in cases:
                fh.write(json.dumps(c) + "\n")
        out.append(path)
    return out


def testcase_path(test_dir: str, task: str, n: int) -> str:
    return os.path.join(test_dir, task, "testcases", f"{n}_{task}.jsonl")


def load_testcases(path: str) -> List[Dict]:
    with open(path) as fh:
        return [json.loads(line) for line in fh if line.strip()]


# ------------------------------------------------------------------------------------------------ scoring
def parse_number(text: str) -> int:
    """The last integer in the model's output, -1 when there is none (the reference's rule, longeval.py:243-248)."""
    found = re.findall(r"\d+", text)
    return int(found[-1]) if found else -1


def output_dir_for(model_name_or_path: str, task: str, root: str = "evaluation") -> str:
    name = model_name_or_path.rstrip("/").split("/")[-1]
    path = os.path.join(root, task, "predictions", name)
    os.makedirs(path, exist_ok=True)
    return path


def _answer(model, tokenizer, prompt: str, max_new_tokens: int, use_cache: bool) -> Tuple[str, int]:
    from .generation import generate
    rec = generate(model, tokenizer, [prompt], maximum_tokens=max_new_tokens, temperature=0.0, use_cache=use_cache)[0]
    return rec["text"], len(tokenizer.tokenize(prompt))


def test_lines_one_sample(model, tokenizer, case: Dict, output_file: str, idx: int, max_new_tokens: int = 32,
                          use_cache: bool = True):
    text, plen = _answer(model, tokenizer, case["prompt"], max_new_tokens, use_cache)
    got = parse_number(text)
    summary = f"Label: {case['expected_number']}, Predict: {text}, Parsed: {got}, prompt length: {plen}".replace("\n", " ")
    with open(output_file, "w" if idx == 0 else "a") as fh:
        fh.write(summary + "\n")
    return got == case["expected_number"], plen, summary


def test_topics_one_sample(model, tokenizer, case: Dict, output_file: str, idx: int, max_new_tokens: int = 50,
                           use_cache: bool = True):
    text, plen = _answer(model, tokenizer, case["prompt"], max_new_tokens, use_cache)
    summary = f"Label: {case['topics'][0]}, Predict: {text}, prompt length: {plen}".replace("\n", " ")
    with open(output_file, "w" if idx == 0 else "a") as fh:
        fh.write(summary + "\n")
    return None, plen, summary


def longeval_test(model, tokenizer, output_dir: str, task: str, test_dir: str, eval_shortest_only: bool = False,
                  sizes: Optional[Iterable[int]] = None, use_cache: bool = True, max_cases: Optional[int] = None) -> Dict[int, Dict]:
    """Runs every size of a task; returns {size: {"accuracy" (lines only), "avg_prompt_length", "cases"}}."""
    if task not in ("lines", "topics"):
        raise ValueError(f"unsupported task {task!r}")
    sizes = tuple(sizes) if sizes else (LINES_SIZES if task == "lines" else TOPICS_SIZES)
    results = {}
    for n in sizes:
        cases = load_testcases(testcase_path(test_dir, task, n))
        if max_cases:
            cases = cases[:max_cases]
        out_file = os.path.join(output_dir, f"{n}_response.txt")
        correct, avg = 0, 0.0
        for idx, case in enumerate(cases):
            fn = test_lines_one_sample if task == "lines" else test_topics_one_sample
            ok, plen, _ = fn(model, tokenizer, case, out_file, idx, use_cache=use_cache)
            correct += bool(ok)
            avg += plen / max(len(cases), 1)
        res = {"avg_prompt_length": avg, "cases": len(cases)}
        if task == "lines":
            res["accuracy"] = correct / max(len(cases), 1)
            with open(out_file, "a") as fh:
                fh.write(f"Accuracy: {res['accuracy']}")
        results[n] = res
        print(f"finished {n} {task} per prompt: average prompt length {avg:.0f}"
              + (f", accuracy {res['accuracy']:.3f}" if task == "lines" else ""))
        if eval_shortest_only:
            break
    return results


def main(argv=None):
    ap = argparse.ArgumentParser(description="LongEval lines / topics tasks for a checkpoint of this framework")
    ap.add_argument("--model-name-or-path", required=True, help="checkpoint directory (a save root or a global_step directory)")
    ap.add_argument("--config", nargs="*", default=None, help="YAML files (default: the copies stored with the checkpoint)")
    ap.add_argument("--task", required=True, choices=["lines", "topics"])
    ap.add_argument("--test-dir", default="evaluation", help="directory holding <task>/testcases/*.jsonl")
    ap.add_argument("--make-testcases", type=int, default=0, metavar="N", help="first write N synthetic cases per size")
    ap.add_argument("--sizes", type=int, nargs="*", default=None)
    ap.add_argument("--eval-shortest-only", action="store_true")
    ap.add_argument("--no-cache", action="store_true", help="recompute the context every generated token")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.make_testcases:
        write_testcases(a.test_dir, a.task, a.sizes, a.make_testcases, a.seed)
    from .load import load_for_inference
    model, tokenizer, _ = load_for_inference(a.model_name_or_path, a.config)
    out = output_dir_for(a.model_name_or_path, a.task)
    print(f"output to {out}")
    return longeval_test(model, tokenizer, out, a.task, a.test_dir, a.eval_shortest_only, a.sizes, not a.no_cache)


if __name__ == "__main__":
    main()
