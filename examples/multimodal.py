"""An image in the prompt: as encoder input for the model's vision tower (patches + their grid) or as ready embeddings.

    python examples/multimodal.py --device cpu          # tiny random-weight Qwen2-VL-style model
    python examples/multimodal.py --model /path/to/Qwen2-VL-checkpoint
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from onecat_vllm import LLM, SamplingParams  # noqa: E402

from _tiny import parse  # noqa: E402

IMG = 250
TINY_VL = dict(architectures=["Qwen2VLForConditionalGeneration"], hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
               num_key_value_heads=2, head_dim=16, vocab_size=300, max_position_embeddings=1024, image_token_id=IMG,
               rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]},
               vision_config=dict(depth=2, embed_dim=32, hidden_size=64, num_heads=4, mlp_ratio=2, patch_size=4, spatial_merge_size=2,
                                  temporal_patch_size=2, in_channels=3))

if __name__ == "__main__":
    args = parse(__doc__)
    if args.model:
        llm = LLM(model=args.model, device=args.device, max_model_len=2048)
        image_id = llm.llm_engine.cfg.model_config.mm_token_ids["image"]
        patch_dim, hidden = 3 * 2 * 14 * 14, llm.llm_engine.cfg.model_config.hidden_size
    else:
        llm = LLM(hf_config=TINY_VL, device=args.device, dtype="float32" if args.device == "cpu" else "bfloat16", max_model_len=512)
        image_id, patch_dim, hidden = IMG, 3 * 2 * 4 * 4, 64
    sp = SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True)
    t, h, w = 1, 4, 6                                     # 24 patches -> 6 embedding positions on a 2 x 3 grid
    pixels = {"pixel_values": torch.randn(t * h * w, patch_dim), "image_grid_thw": (t, h, w)}
    a = llm.generate([{"prompt_token_ids": [5, 6, image_id, 7, 8], "multi_modal_data": {"image": pixels}}], sp)[0]
    print("pixels     ->", a.outputs[0].token_ids)
    embeds = torch.randn(6, hidden) * 0.02                # the same placeholder filled with ready embeddings (6 positions)
    b = llm.generate([{"prompt_token_ids": [5, 6, image_id, 7, 8], "multi_modal_data": {"image": embeds}}], sp)[0]
    print("embeddings ->", b.outputs[0].token_ids)
    llm.shutdown()
