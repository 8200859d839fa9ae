"""A user logits processor for the tests: bans the token ids listed in ``SamplingParams.extra_args["banned"]`` and, for requests
that ask for it with ``extra_args["force"]``, leaves only that token."""
import torch


class BanOrForce:
    def __init__(self, vllm_config, device):
        self.vocab = vllm_config.model_config.vocab_size
        self.calls = 0

    def apply(self, logits: torch.Tensor, rows: list) -> torch.Tensor:
        self.calls += 1
        for i, r in enumerate(rows):
            ex = r["extra_args"]
            if ex.get("banned"):
                logits[i, torch.tensor(ex["banned"], device=logits.device)] = -float("inf")
            if ex.get("force") is not None and len(r["output_token_ids"]) % 2 == 1:   # every second generated token
                keep = logits[i, ex["force"]].clone()
                logits[i] = -float("inf")
                logits[i, ex["force"]] = keep
        return logits
