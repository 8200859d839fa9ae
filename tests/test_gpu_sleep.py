"""Sleep mode on a GPU: device memory really goes back to the driver, tensors keep their addresses, offloaded contents return."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pools_release_memory_and_keep_addresses():
    from onecat_vllm.utils.cumem import CuMemAllocator
    a = CuMemAllocator.get()
    with a.use_memory_pool("weights"):
        w = torch.randn(64 << 20, device="cuda", dtype=torch.bfloat16)      # 128 MiB
    with a.use_memory_pool("kv_cache"):
        kv = torch.zeros(128 << 20, device="cuda", dtype=torch.uint8)       # 128 MiB
    keep = w.float().sum().item()
    ptrs = (w.data_ptr(), kv.data_ptr())
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    freed = a.sleep(offload_tags=("weights",), discard_tags=("kv_cache",))
    free1, _ = torch.cuda.mem_get_info()
    assert freed >= 256 << 20 and free1 - free0 >= 200 << 20, (freed, free1 - free0)
    assert a.stats()["host_backup_bytes"] >= 128 << 20
    a.wake_up(("weights",))
    assert w.data_ptr() == ptrs[0] and w.float().sum().item() == keep
    a.wake_up(("kv_cache",))
    kv.fill_(3)
    torch.cuda.synchronize()
    assert kv.data_ptr() == ptrs[1] and int(kv[-1]) == 3 and a.stats()["asleep_bytes"] == 0
    free2, _ = torch.cuda.mem_get_info()
    assert free0 - free2 < 64 << 20


@pytest.mark.timeout(600)
def test_engine_sleeps_and_wakes_with_the_same_outputs(tmp_path):
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, save_pretrained
    from onecat_vllm.models import build_model
    cfg = dict(architectures=["Qwen3ForCausalLM"], hidden_size=1024, intermediate_size=2048, num_hidden_layers=3, num_attention_heads=8,
               num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048, max_position_embeddings=2048,
               tie_word_embeddings=False)
    m = build_model(ModelConfig.from_hf_dict(cfg, dtype=torch.bfloat16), "cpu")
    dummy_init(m, 0, std=0.05)
    save_pretrained(m, cfg, str(tmp_path))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (5, 40, 64)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    llm = LLM(model=str(tmp_path), device="cuda", dtype="bfloat16", max_model_len=512, max_num_seqs=8, gpu_memory_utilization=0.2,
              enable_sleep_mode=True)
    ref = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]
    free0, _ = torch.cuda.mem_get_info()
    llm.sleep(1)
    free1, _ = torch.cuda.mem_get_info()
    assert free1 - free0 > 1 << 30, "the KV cache alone is several GiB: sleeping must return it"
    llm.wake_up()
    again = [o.outputs[0].token_ids for o in llm.generate(prompts, sp)]   # decode graphs captured before the sleep replay on the same addresses
    llm.shutdown()
    assert again == ref
