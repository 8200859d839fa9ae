"""Weight hand-over by broadcast over a group of its own (gloo ranks on CPU): a trainer process (rank 0) sends a new state dict, a
worker holding a live engine (rank 1) loads it in place and its greedy output changes to that of the new weights."""
import torch
import torch.multiprocessing as mp

CFG = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=1e4)


def _trainer(port, q):
    from onecat_vllm.config import ModelConfig
    from onecat_vllm.loader.weights import dummy_init, to_hf_state_dict
    from onecat_vllm.models import build_model
    from onecat_vllm.utils.weight_transfer import BroadcastWeightTransfer
    m = build_model(ModelConfig.from_hf_dict(CFG, dtype=torch.float32), "cpu")
    dummy_init(m, 123)
    named = list(to_hf_state_dict(m).items())
    eng = BroadcastWeightTransfer.init(f"tcp://127.0.0.1:{port}", 0, 2, "cpu", bucket_bytes=1 << 16)
    q.put(eng.describe(named))
    eng.send(named)
    eng.close()


def test_broadcast_weight_update_changes_a_live_engine():
    from onecat_vllm import LLM, SamplingParams
    from onecat_vllm.executor.multiproc import _free_port
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    prompt = [list(range(5, 25))]
    llm = LLM(hf_config=CFG, device="cpu", dtype="float32", max_model_len=128, seed=0, enable_prefix_caching=False)
    before = llm.generate(prompt, sp)[0].outputs[0].token_ids
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    p = ctx.Process(target=_trainer, args=(port, q))
    p.start()
    try:
        assert llm.collective_rpc("init_weight_transfer", args=(f"tcp://127.0.0.1:{port}", 1, 2)) == [True]
        meta = q.get(timeout=60)
        n = llm.collective_rpc("update_weights_broadcast", args=(meta,))[0]
        assert n > 0
    finally:
        p.join(60)
    after = llm.generate(prompt, sp)[0].outputs[0].token_ids
    llm.shutdown()
    ref = LLM(hf_config=CFG, device="cpu", dtype="float32", max_model_len=128, seed=123, enable_prefix_caching=False)
    want = ref.generate(prompt, sp)[0].outputs[0].token_ids
    ref.shutdown()
    assert after != before and after == want
