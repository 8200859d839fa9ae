"""Benchmark datasets and parameter sweeps (CPU only: the client runner and the server are stand-ins)."""
import argparse
import json

import pytest

from onecat_vllm.entrypoints import bench_datasets as D
from onecat_vllm.entrypoints import bench_sweep as S


def _args(**kw):
    base = dict(seed=0, num_prompts=8, input_len=32, output_len=16, dataset_name="random", dataset_path=None, random_prefix_len=0,
                random_range_ratio=0.0, prefix_repetition_num_prefixes=2, prefix_repetition_prefix_len=16, sonnet_prefix_len=10,
                hub_prompt_field="prompt", burstgpt_model="GPT-4", trace_block_size=8, no_oversample=False)
    base.update(kw)
    return argparse.Namespace(**base)


def test_random_dataset_prefix_and_range():
    rows = D.build_dataset(_args(random_prefix_len=5, random_range_ratio=0.5), vocab=100)
    assert len(rows) == 8
    assert all(r.prompt[:5] == rows[0].prompt[:5] for r in rows)
    assert all(5 + 16 <= r.prompt_len <= 5 + 48 and 8 <= r.expected_output_len <= 24 for r in rows)
    assert D.build_dataset(_args(random_prefix_len=5, random_range_ratio=0.5), vocab=100)[3].prompt == rows[3].prompt  # seeded


def test_prefix_repetition_shares_exactly_the_prefixes():
    rows = D.build_dataset(_args(dataset_name="prefix_repetition"), vocab=1000)
    heads = {tuple(r.prompt[:16]) for r in rows}
    assert len(heads) == 2 and all(r.prompt_len == 32 for r in rows)


def test_sharegpt_filters_and_oversamples(tmp_path):
    data = [{"conversations": [{"value": "tell me a long story about cats"}, {"value": "once upon a time there was"}]},
            {"conversations": [{"value": "hi"}, {"value": "hello there friend again"}]},  # prompt too short
            {"conversations": [{"value": "only one turn here"}]}]
    p = tmp_path / "s.json"
    p.write_text(json.dumps(data))
    rows = D.build_dataset(_args(dataset_name="sharegpt", dataset_path=str(p), num_prompts=3), vocab=10)
    assert len(rows) == 3 and all(r.prompt.startswith("tell me") and r.expected_output_len == 6 for r in rows)
    assert len(D.build_dataset(_args(dataset_name="sharegpt", dataset_path=str(p), num_prompts=3, no_oversample=True), vocab=10)) == 1


def test_sonnet_custom_hub(tmp_path):
    poem = tmp_path / "poem.txt"
    poem.write_text("\n".join(f"line {i} of the poem goes here" for i in range(20)))
    rows = D.build_dataset(_args(dataset_name="sonnet", dataset_path=str(poem), input_len=60, sonnet_prefix_len=25, num_prompts=4), vocab=10)
    assert len(rows) == 4 and all(40 <= r.prompt_len <= 70 and r.expected_output_len == 16 for r in rows)
    first = rows[0].prompt.splitlines()[1]
    assert all(r.prompt.splitlines()[1] == first for r in rows)  # the shared prefix lines
    cu = tmp_path / "c.jsonl"
    cu.write_text('{"prompt": "a b c", "output_tokens": 7}\n{"prompt": "d e"}\n')
    got = sorted(D.build_dataset(_args(dataset_name="custom", dataset_path=str(cu), num_prompts=2), vocab=10), key=lambda r: r.prompt)
    assert [(r.prompt_len, r.expected_output_len) for r in got] == [(3, 7), (2, 16)]
    hub = tmp_path / "h.json"
    hub.write_text(json.dumps([{"turns": ["write a poem", "again"]}]))
    assert D.build_dataset(_args(dataset_name="hub", dataset_path=str(hub), hub_prompt_field="turns.0", num_prompts=1), vocab=10)[0].prompt == "write a poem"
    with pytest.raises(ValueError):
        D.build_dataset(_args(dataset_name="custom"), vocab=10)


def test_traces_keep_arrivals_and_shared_blocks(tmp_path):
    b = tmp_path / "b.csv"
    b.write_text("Timestamp,Model,Request tokens,Response tokens\n10,GPT-4,12,5\n4,GPT-4,6,3\n7,ChatGPT,9,9\n")
    rows = D.build_dataset(_args(dataset_name="burstgpt", dataset_path=str(b), num_prompts=2), vocab=50)
    assert [(r.prompt_len, r.expected_output_len, r.arrival_s) for r in rows] == [(6, 3, 0.0), (12, 5, 6.0)]
    t = tmp_path / "t.jsonl"
    t.write_text('{"timestamp": 0, "input_length": 20, "output_length": 4, "hash_ids": [1, 2]}\n'
                 '{"timestamp": 500, "input_length": 18, "output_length": 2, "hash_ids": [1, 3]}\n')
    rows = D.build_dataset(_args(dataset_name="timed_trace", dataset_path=str(t), num_prompts=2), vocab=50)
    assert rows[0].prompt[:8] == rows[1].prompt[:8] and rows[0].prompt[8:16] != rows[1].prompt[8:16]
    assert [r.prompt_len for r in rows] == [20, 18] and rows[1].arrival_s == 0.5


def test_param_sets_and_command_overrides():
    assert S.load_param_sets(None) == [{}]
    assert S.load_param_sets('{"a": [1, 2], "b": "x"}') == [{"a": 1, "b": "x"}, {"a": 2, "b": "x"}]
    named = S.load_param_sets('{"fast": {"a": 1}, "slow": {"a": 2}}')
    assert [S.set_name(n) for n in named] == ["fast", "slow"]
    cmd = ["srv", "--max-num-seqs", "8", "--flag", "--x=1", "--keep", "k"]
    got = S.apply_params(cmd, {"max_num_seqs": 64, "flag": False, "x": 2, "new_flag": True, "_name": "n"})
    assert got == ["srv", "--keep", "k", "--max-num-seqs", "64", "--x", "2", "--new-flag"]


class _FakeServer:
    started = []

    def __init__(self, cmd, *a):
        self.cmd = cmd
        self.resets = 0

    def __enter__(self):
        _FakeServer.started.append(self.cmd)
        return self

    def __exit__(self, *e):
        return False

    def reset_caches(self):
        self.resets += 1


def _fake_client(calls):
    def run(cmd, path, show):
        calls.append(cmd)
        conc = int(cmd[cmd.index("--max-concurrency") + 1]) if "--max-concurrency" in cmd else 4
        rate = float(cmd[cmd.index("--request-rate") + 1]) if "--request-rate" in cmd else None
        thr = min(conc, 16) * 2.0 if rate is None else min(rate, 32.0)
        return {"request_throughput": thr, "mean_e2el_ms": 500.0, "output_throughput": thr * 10, "p50_tpot_ms": 10.0 + conc}
    return run


def test_grid_runs_resume_and_summary(tmp_path):
    _FakeServer.started = []
    calls = []
    kw = dict(run_client=_fake_client(calls), server_factory=_FakeServer)
    rows = S.run_grid(["srv"], ["cli"], [{"tp": 1}, {"tp": 2}], [{"max_concurrency": 1}, {"max_concurrency": 8}], tmp_path, 2, **kw)
    assert len(rows) == 8 and len(calls) == 8 and len(_FakeServer.started) == 2
    assert _FakeServer.started[1] == ["srv", "--tp", "2"]
    assert (tmp_path / "tp=2" / "max_concurrency=8" / "run=1.json").exists()
    # everything is on disk: a resumed sweep starts no server and runs no client
    again = S.run_grid(["srv"], ["cli"], [{"tp": 1}, {"tp": 2}], [{"max_concurrency": 1}, {"max_concurrency": 8}], tmp_path, 2, resume=True, **kw)
    assert len(again) == 8 and len(calls) == 8 and len(_FakeServer.started) == 2
    summ = S.write_summary(rows, tmp_path)
    assert summ["runs"] == 8 and [r["max_concurrency"] for r in summ["pareto"]] == [1, 8]
    assert (tmp_path / "summary.csv").read_text().count("\n") == 9


def test_workload_explorer_spaces_points_between_serial_and_saturated(tmp_path):
    calls = []
    rows = S.explore_workload(["cli"], {}, {"num_prompts": 64}, tmp_path, 1, "request_rate", 4, 64, run_client=_fake_client(calls))
    # serial reaches 2 req/s, the saturated run 32 req/s; two points go between them
    rates = [float(c[c.index("--request-rate") + 1]) for c in calls if "--request-rate" in c]
    assert rates == [12.0, 22.0] and len(rows) == 4
    with pytest.raises(ValueError):
        S.explore_workload(["cli"], {}, {}, tmp_path, 1, "request_rate", 1, 64)


def test_dry_run_prints_commands_only(tmp_path, capsys):
    rows = S.run_grid(["srv", "--port", "9"], ["cli"], [{"a": 1}], [{"b": 2}], tmp_path, 1, dry_run=True)
    out = capsys.readouterr().out
    assert rows == [] and "srv --port 9 --a 1" in out and "cli --b 2 --save-result" in out and not list(tmp_path.iterdir())
    assert S.ServerProcess(["srv", "--port", "9"]).address() == "http://127.0.0.1:9"
