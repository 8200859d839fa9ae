"""Workloads for the benchmark harness: every dataset yields ``SampleRequest`` rows (prompt, prompt length, wanted output
length) from a local file or a seeded generator; nothing is downloaded
(reference: vllm/benchmarks/datasets/datasets.py ``SampleRequest``:76, ``RandomDataset``:534, ``ShareGPTDataset``:1317,
``TimedTrace``:1407, ``CustomDataset``:2409, ``SonnetDataset``:2924, ``BurstGPTDataset``:3012,
``PrefixRepetitionRandomDataset``:4081; the hub-backed sets need a network and are represented by ``HubDataset`` reading the same
records from a local JSON/JSONL export)."""
from __future__ import annotations

import csv
import json
import random
from dataclasses import dataclass
from typing import Callable, Optional, Sequence, Union

Prompt = Union[str, list]


@dataclass
class SampleRequest:
    prompt: Prompt  # text, or token ids when the dataset is synthetic
    prompt_len: int
    expected_output_len: int
    arrival_s: Optional[float] = None  # traces carry their own arrival times
    request_id: Optional[str] = None


class _WordTokenizer:
    """Stand-in when no tokenizer is given: one token per whitespace-separated word."""

    def encode(self, text: str) -> list:
        return text.split()


def _count(tok, text: str) -> int:
    return len(tok.encode(text))


class BenchmarkDataset:
    """``sample(n)`` returns exactly ``n`` rows; a set with fewer rows repeats (oversampling) unless ``no_oversample``."""

    name = "base"

    def __init__(self, seed: int = 0, tokenizer=None, no_oversample: bool = False):
        self.rng = random.Random(seed)
        self.tok = tokenizer or _WordTokenizer()
        self.no_oversample = no_oversample

    def rows(self) -> list[SampleRequest]:
        raise NotImplementedError

    def sample(self, n: int) -> list[SampleRequest]:
        rows = self.rows()
        if not rows:
            raise ValueError(f"dataset {self.name!r} produced no usable rows")
        if len(rows) >= n:
            return rows[:n]
        if self.no_oversample:
            return rows
        out = list(rows)
        while len(out) < n:
            src = self.rng.choice(rows)
            out.append(SampleRequest(src.prompt, src.prompt_len, src.expected_output_len, src.arrival_s))
        return out


def _ranged(rng: random.Random, mean: int, ratio: float) -> int:
    if ratio <= 0:
        return max(int(mean), 1)
    return max(rng.randint(int(mean * (1 - ratio)), int(mean * (1 + ratio))), 1)


class RandomDataset(BenchmarkDataset):
    """Uniform token ids; ``prefix_len`` tokens are shared by every prompt; lengths vary by ``range_ratio`` around the means."""

    name = "random"

    def __init__(self, n: int, input_len: int, output_len: int, vocab: int, prefix_len: int = 0, range_ratio: float = 0.0, **kw):
        super().__init__(**kw)
        self.n, self.input_len, self.output_len, self.vocab = n, input_len, output_len, vocab
        self.prefix_len, self.range_ratio = prefix_len, range_ratio

    def rows(self):
        prefix = [self.rng.randrange(self.vocab) for _ in range(self.prefix_len)]
        out = []
        for _ in range(self.n):
            il, ol = _ranged(self.rng, self.input_len, self.range_ratio), _ranged(self.rng, self.output_len, self.range_ratio)
            ids = prefix + [self.rng.randrange(self.vocab) for _ in range(il)]
            out.append(SampleRequest(ids, len(ids), ol))
        return out


class PrefixRepetitionDataset(BenchmarkDataset):
    """``num_prefixes`` distinct prefixes, each followed by fresh suffixes: the prefix-cache hit rate is set by construction."""

    name = "prefix_repetition"

    def __init__(self, n: int, prefix_len: int, suffix_len: int, num_prefixes: int, output_len: int, vocab: int, **kw):
        super().__init__(**kw)
        self.n, self.prefix_len, self.suffix_len, self.num_prefixes, self.output_len, self.vocab = n, prefix_len, suffix_len, num_prefixes, output_len, vocab

    def rows(self):
        prefixes = [[self.rng.randrange(self.vocab) for _ in range(self.prefix_len)] for _ in range(max(self.num_prefixes, 1))]
        out = []
        for i in range(self.n):
            ids = prefixes[i % len(prefixes)] + [self.rng.randrange(self.vocab) for _ in range(self.suffix_len)]
            out.append(SampleRequest(ids, len(ids), self.output_len))
        self.rng.shuffle(out)
        return out


class ShareGPTDataset(BenchmarkDataset):
    """A ShareGPT JSON export: the first turn is the prompt; the second turn's length is the wanted output length unless
    ``output_len`` fixes it. Rows shorter than 4 tokens on either side or longer than ``max_total`` are dropped."""

    name = "sharegpt"

    def __init__(self, path: str, output_len: Optional[int] = None, max_prompt: int = 1024, max_total: int = 2048, **kw):
        super().__init__(**kw)
        self.path, self.output_len, self.max_prompt, self.max_total = path, output_len, max_prompt, max_total

    def rows(self):
        with open(self.path) as f:
            data = json.load(f)
        data = [d for d in data if len(d.get("conversations", d.get("conversation", []))) >= 2]
        self.rng.shuffle(data)
        out = []
        for d in data:
            conv = d.get("conversations", d.get("conversation"))
            prompt, completion = conv[0]["value"], conv[1]["value"]
            pl = _count(self.tok, prompt)
            ol = self.output_len if self.output_len is not None else _count(self.tok, completion)
            if pl < 4 or (self.output_len is None and ol < 4) or pl > self.max_prompt or pl + ol > self.max_total:
                continue
            out.append(SampleRequest(prompt, pl, ol))
        return out


class SonnetDataset(BenchmarkDataset):
    """Prompts assembled from the lines of a poem file: a fixed prefix of lines shared by all prompts, then randomly drawn
    lines until the prompt reaches ``input_len`` tokens."""

    name = "sonnet"

    def __init__(self, path: str, n: int, input_len: int = 550, prefix_len: int = 200, output_len: int = 150, **kw):
        super().__init__(**kw)
        if prefix_len > input_len:
            raise ValueError("sonnet: prefix_len must not exceed input_len")
        self.path, self.n, self.input_len, self.prefix_len, self.output_len = path, n, input_len, prefix_len, output_len

    def rows(self):
        with open(self.path) as f:
            lines = [ln for ln in f.read().splitlines() if ln.strip()]
        if not lines:
            return []
        avg = max(sum(_count(self.tok, ln) for ln in lines) / len(lines), 1.0)
        head = "Pick as many lines as you can from these poem lines:\n"
        base = _count(self.tok, head)
        n_prefix = max(int((self.prefix_len - base) / avg), 0)
        n_input = max(int((self.input_len - base) / avg), n_prefix + 1)
        prefix = lines[:n_prefix]
        out = []
        for _ in range(self.n):
            extra = [self.rng.choice(lines) for _ in range(n_input - n_prefix)]
            text = head + "\n".join(prefix + extra)
            out.append(SampleRequest(text, _count(self.tok, text), self.output_len))
        return out


class CustomDataset(BenchmarkDataset):
    """A JSONL file with one ``{"prompt": ..., "output_tokens": optional}`` object per line."""

    name = "custom"

    def __init__(self, path: str, output_len: int = 256, **kw):
        super().__init__(**kw)
        self.path, self.output_len = path, output_len

    def rows(self):
        out = []
        with open(self.path) as f:
            for ln in f:
                ln = ln.strip()
                if not ln:
                    continue
                d = json.loads(ln)
                if "prompt" not in d:
                    raise ValueError("custom dataset rows need a 'prompt' field")
                out.append(SampleRequest(d["prompt"], _count(self.tok, d["prompt"]), int(d.get("output_tokens", self.output_len))))
        self.rng.shuffle(out)
        return out


class HubDataset(CustomDataset):
    """A local JSON/JSONL export of a hub conversation or instruction set. ``prompt_field`` is a dotted path into each record
    (``turns.0``, ``conversations.0.value``, ``question``); the hub itself is not reachable from an air-gapped host."""

    name = "hub"

    def __init__(self, path: str, prompt_field: str = "prompt", output_len: int = 256, **kw):
        super().__init__(path, output_len, **kw)
        self.prompt_field = prompt_field

    def _pick(self, rec):
        cur = rec
        for part in self.prompt_field.split("."):
            cur = cur[int(part)] if isinstance(cur, list) else cur[part]
        return cur

    def rows(self):
        with open(self.path) as f:
            text = f.read().strip()
        recs = json.loads(text) if text.startswith("[") else [json.loads(ln) for ln in text.splitlines() if ln.strip()]
        out = []
        for r in recs:
            p = self._pick(r)
            out.append(SampleRequest(p, _count(self.tok, p), self.output_len))
        self.rng.shuffle(out)
        return out


class BurstGPTDataset(BenchmarkDataset):
    """The BurstGPT trace CSV (columns ``Timestamp, Model, Request tokens, Response tokens, …``): synthetic token ids of the logged
    lengths, with the logged arrival times kept so the client can replay the burst pattern."""

    name = "burstgpt"

    def __init__(self, path: str, vocab: int, model_filter: Optional[str] = "GPT-4", **kw):
        super().__init__(**kw)
        self.path, self.vocab, self.model_filter = path, vocab, model_filter

    def rows(self):
        out = []
        with open(self.path, newline="") as f:
            for row in csv.DictReader(f):
                if self.model_filter and row.get("Model") != self.model_filter:
                    continue
                il, ol = int(float(row["Request tokens"])), int(float(row["Response tokens"]))
                if il <= 0 or ol <= 0:
                    continue
                ids = [self.rng.randrange(self.vocab) for _ in range(il)]
                out.append(SampleRequest(ids, il, ol, arrival_s=float(row.get("Timestamp", 0.0) or 0.0)))
        if out:
            t0 = min(r.arrival_s for r in out)
            for r in out:
                r.arrival_s -= t0
            out.sort(key=lambda r: r.arrival_s)
        return out


class TimedTraceDataset(BenchmarkDataset):
    """A JSONL trace ``{"timestamp": ms, "input_length": n, "output_length": m, "hash_ids": [...]}``: each hash id names one
    ``block_size``-token block, so requests that share ids share a prefix of exactly those blocks."""

    name = "timed_trace"

    def __init__(self, path: str, vocab: int, block_size: int = 512, **kw):
        super().__init__(**kw)
        self.path, self.vocab, self.block_size = path, vocab, block_size

    def rows(self):
        blocks: dict = {}
        out = []
        with open(self.path) as f:
            for ln in f:
                if not ln.strip():
                    continue
                d = json.loads(ln)
                ids: list = []
                for h in d.get("hash_ids", []):
                    if h not in blocks:
                        r = random.Random(hash((h, self.vocab)) & 0xFFFFFFFF)
                        blocks[h] = [r.randrange(self.vocab) for _ in range(self.block_size)]
                    ids += blocks[h]
                il = int(d["input_length"])
                ids = ids[:il] + [self.rng.randrange(self.vocab) for _ in range(max(il - len(ids), 0))]
                out.append(SampleRequest(ids, il, int(d["output_length"]), arrival_s=float(d.get("timestamp", 0)) / 1e3))
        out.sort(key=lambda r: r.arrival_s)
        return out


DATASETS: dict[str, Callable] = {c.name: c for c in (RandomDataset, PrefixRepetitionDataset, ShareGPTDataset, SonnetDataset,
                                                      CustomDataset, HubDataset, BurstGPTDataset, TimedTraceDataset)}


def add_dataset_args(p) -> None:
    p.add_argument("--dataset-name", default="random", choices=sorted(DATASETS))
    p.add_argument("--dataset-path", default=None)
    p.add_argument("--random-prefix-len", type=int, default=0)
    p.add_argument("--random-range-ratio", type=float, default=0.0)
    p.add_argument("--prefix-repetition-num-prefixes", type=int, default=8)
    p.add_argument("--prefix-repetition-prefix-len", type=int, default=256)
    p.add_argument("--sonnet-prefix-len", type=int, default=200)
    p.add_argument("--hub-prompt-field", default="prompt")
    p.add_argument("--burstgpt-model", default="GPT-4")
    p.add_argument("--trace-block-size", type=int, default=512)
    p.add_argument("--no-oversample", action="store_true")
    p.add_argument("--replay-arrivals", action="store_true", help="send trace rows at their logged arrival times")


def build_dataset(a, vocab: int, tokenizer=None) -> list[SampleRequest]:
    """The rows the chosen ``--dataset-name`` yields for this run's ``--num-prompts`` / ``--input-len`` / ``--output-len``."""
    kw = dict(seed=getattr(a, "seed", 0), tokenizer=tokenizer, no_oversample=getattr(a, "no_oversample", False))
    name = getattr(a, "dataset_name", "random")
    n = a.num_prompts
    need_path = name not in ("random", "prefix_repetition")
    if need_path and not getattr(a, "dataset_path", None):
        raise ValueError(f"--dataset-name {name} needs --dataset-path")
    if name == "random":
        ds = RandomDataset(n, a.input_len, a.output_len, vocab, getattr(a, "random_prefix_len", 0), getattr(a, "random_range_ratio", 0.0), **kw)
    elif name == "prefix_repetition":
        pl = a.prefix_repetition_prefix_len
        ds = PrefixRepetitionDataset(n, pl, max(a.input_len - pl, 1), a.prefix_repetition_num_prefixes, a.output_len, vocab, **kw)
    elif name == "sharegpt":
        ds = ShareGPTDataset(a.dataset_path, None, **kw)
    elif name == "sonnet":
        ds = SonnetDataset(a.dataset_path, n, a.input_len, a.sonnet_prefix_len, a.output_len, **kw)
    elif name == "custom":
        ds = CustomDataset(a.dataset_path, a.output_len, **kw)
    elif name == "hub":
        ds = HubDataset(a.dataset_path, a.hub_prompt_field, a.output_len, **kw)
    elif name == "burstgpt":
        ds = BurstGPTDataset(a.dataset_path, vocab, a.burstgpt_model or None, **kw)
    else:
        ds = TimedTraceDataset(a.dataset_path, vocab, a.trace_block_size, **kw)
    return ds.sample(n)


def prompt_lens(rows: Sequence[SampleRequest]) -> int:
    return sum(r.prompt_len for r in rows)
