"""Shared by the examples: a tiny random-weight Llama-style configuration, used when no model directory is given."""
import argparse

TINY = dict(architectures=["LlamaForCausalLM"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, vocab_size=258, max_position_embeddings=512, eos_token_id=257)


def parse(description: str) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=description)
    ap.add_argument("--model", default=None, help="checkpoint directory (default: a tiny random-weight model with a byte tokenizer)")
    ap.add_argument("--device", default="auto", help="auto | cuda | cpu")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    return ap.parse_args()


def engine_kwargs(a: argparse.Namespace) -> dict:
    kw = dict(device=a.device, tensor_parallel_size=a.tensor_parallel_size, max_model_len=512)
    if a.model:
        kw.update(model=a.model, tokenizer=a.model)
    else:
        kw.update(hf_config=TINY, tokenizer="byte", dtype="float32" if a.device == "cpu" else "bfloat16")
    return kw
