"""Platform description and the local usage record."""
import json

import pytest
import torch

from onecat_vllm import platforms


def test_cpu_platform_and_usage_record(tmp_path, monkeypatch):
    p = platforms.current_platform(refresh=True)
    if not torch.cuda.is_available():
        assert p.is_cpu() and p.dispatch_key == "ref" and not p.supports_native_kernels() and p.default_dtype() == torch.float32
        assert platforms.resolve_device("auto") == "cpu"
        with pytest.raises(ValueError):
            platforms.resolve_device("cuda")
    d = p.describe()
    assert d["device_type"] == p.device_type and d["total_memory"] > 0
    out = tmp_path / "usage.jsonl"
    monkeypatch.setenv("ONECAT_USAGE_STATS_FILE", str(out))
    rec = platforms.usage_record("LLM_CLASS", "LlamaForCausalLM", {"tensor_parallel_size": 2})
    line = json.loads(out.read_text().strip())
    assert line["architecture"] == "LlamaForCausalLM" and line["tensor_parallel_size"] == 2 and line["platform"] == rec["platform"]
