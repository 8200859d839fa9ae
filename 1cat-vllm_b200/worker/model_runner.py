"""Model runner: persistent request state → flat step inputs → forward → logits → sampling / verification →
draft proposal (reference: vllm/v1/worker/gpu_model_runner.py:1091 class, :2182 ``_update_states``, :4705
``_prepare_inputs``, :5159 ``_build_attention_metadata``, :8051 ``execute_model``, :8576 ``sample_tokens``, :9331
``propose_draft_token_ids``; gpu_input_batch.py:92; block_table.py:18,466).

The same class runs on CPU (torch ops, fp32) and on a B200 (hand-written kernels, pinned staging buffers, CUDA
graphs for uniform decode batches). Each step copies that step's inputs host→device from pinned memory and reads
the sampled ids back, so a step timed end to end includes both transfers.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from onecat_vllm.config import VllmConfig
from onecat_vllm.core.kv_cache_utils import KVCacheConfig, KVCacheSpec
from onecat_vllm.core.sched_output import ModelRunnerOutput, SchedulerOutput
from onecat_vllm.logger import init_logger
from onecat_vllm.ops import ref as ref_ops
from onecat_vllm.parallel import state as ps
from onecat_vllm.sample.metadata import SamplingMetadata
from onecat_vllm.sample.rejection_sampler import RejectionSampler
from onecat_vllm.sample.sampler import Sampler, SamplerOutput, to_logprobs_lists
from onecat_vllm.worker.attn_metadata import AttentionMetadata

log = init_logger(__name__)


@dataclass
class CachedRequestState:
    req_id: str
    token_ids: list  # prompt + outputs known to the runner
    num_prompt_tokens: int
    sampling_params: object
    block_ids: list
    num_computed_tokens: int
    state_slot: int = -1
    generator: Optional[torch.Generator] = None
    eos_token_id: Optional[int] = None
    pooling_params: object = None
    lora_request: object = None
    prompt_embeds: Optional[torch.Tensor] = None
    mm_features: Optional[list] = None  # multimodal items of the prompt (placeholder ranges + encoder inputs)
    pool_sum: Optional[torch.Tensor] = None  # running sum of hidden states (mean pooling over a chunked prompt)
    pool_first: Optional[torch.Tensor] = None  # hidden state of the first token (cls pooling)
    pending: int = 0  # tokens sampled by a step that is still in flight (async scheduling): on the device, not yet in token_ids
    mrope: object = None  # int32 [3, prompt] rotary positions of a multimodal prompt (models with rotary sections), built on first use
    mrope_delta: int = 0  # what a generated token adds to its index to get its (three equal) rotary positions


class _Ready:
    """Stands in for a CUDA event on the CPU path, where the copy has completed by the time it returns."""

    def synchronize(self) -> None:
        pass


@dataclass
class PendingStep:
    """A launched step whose sampled tokens have not been read back yet."""
    out: "ModelRunnerOutput"
    rows: Optional[list] = None        # logits rows per request (1 where the request sampled)
    n: int = 0                         # sampled tokens on their way to ``host``
    host: Optional[torch.Tensor] = None
    done: object = None                # event recorded after the device-to-host copy
    ev: Optional[tuple] = None         # (start, end) timing events
    status: Optional[torch.Tensor] = None  # pinned words the kernels' status was copied into behind the step


class ModelRunner:
    def __init__(self, vllm_config: VllmConfig, device: torch.device):
        self.cfg = vllm_config
        self.mc = vllm_config.model_config
        self.device = device
        self.use_cuda = device.type == "cuda"
        self.block_size = vllm_config.cache_config.block_size
        self.max_model_len = self.mc.max_model_len
        self.max_num_tokens = vllm_config.scheduler_config.max_num_batched_tokens
        self.max_num_reqs = vllm_config.scheduler_config.max_num_seqs
        self.requests: dict[str, CachedRequestState] = {}
        self.model = None
        self.mtp = None
        self.draft = None          # speculative method draft_model: a second CausalLM and its K/V pages
        self.draft_caches = None
        self.kv_caches: list = []
        self._pending_saves: list = []
        self.lora_manager = None
        self.mtp_cache = None
        self.sampler = Sampler()
        sc = vllm_config.speculative_config
        self.spec = sc
        self.num_spec = sc.num_speculative_tokens if sc.enabled else 0
        self.pp = ps.get_state()  # pipeline coordinates of this rank
        self.rejection_sampler = RejectionSampler(sc.conditional_rates(), sc.synthetic_seed) if sc.enabled else None
        self.proposer = None
        self.graphs = None  # worker.cuda_graphs.DecodeGraphs
        self.encoder_cache: dict = {}  # content hash of a multimodal item -> its encoder output [positions, hidden]
        self._last_step_ms = 0.0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self.kernel_launches = 0

    # ------------------------------------------------------------------ model / cache set-up
    def load_model(self) -> None:
        from onecat_vllm.loader.weights import load_model
        t0 = time.time()
        self.model = load_model(self.mc, self.device)
        if self.spec.method == "mtp":
            from onecat_vllm.loader.weights import dummy_init, process_weights_after_loading
            from onecat_vllm.models.decoder import MTPHead
            with torch.device(self.device):
                self.mtp = MTPHead(self.mc, self.model, self.device)
            dummy_init(self.mtp, self.mc.seed + 1)
            if self.mc.load_format != "dummy" and os.path.isdir(self.mc.model):
                from onecat_vllm.loader.weights import load_mtp_weights
                n = load_mtp_weights(self.mtp, self.mc)
                if n == 0:
                    log.warning_once("the checkpoint has no multi-token-prediction tensors: the draft head runs with random weights")
            process_weights_after_loading(self.mtp)
            self.mtp.eval()
        if self.spec.method == "eagle":
            # the drafting loop is the MTP one: the head sits in the same slot
            from onecat_vllm.loader.weights import dummy_init, load_eagle_weights, process_weights_after_loading
            from onecat_vllm.models.decoder import EagleHead
            with torch.device(self.device):
                self.mtp = EagleHead(self.mc, self.model, self.device)
            dummy_init(self.mtp, self.mc.seed + 1)
            if self.spec.model and os.path.isdir(self.spec.model):
                load_eagle_weights(self.mtp, self.spec.model)
            process_weights_after_loading(self.mtp)
            self.mtp.eval()
        if self.spec.method == "draft_model":
            import dataclasses
            from onecat_vllm.config import ModelConfig
            from onecat_vllm.loader.weights import load_model
            if not (self.spec.model and os.path.isdir(self.spec.model)):
                raise ValueError("speculative method draft_model needs speculative_config.model = the draft model's checkpoint directory")
            dcfg = ModelConfig.from_pretrained(self.spec.model, dtype=self.mc.dtype, seed=self.mc.seed)
            dcfg.max_model_len = self.mc.max_model_len
            if dcfg.vocab_size != self.mc.vocab_size:
                raise ValueError(f"the draft model's vocabulary ({dcfg.vocab_size}) differs from the target's ({self.mc.vocab_size})")
            if dcfg.is_hybrid or dcfg.use_mla:
                raise ValueError("the draft model must be a plain attention decoder (its K/V pages live under the target's block ids)")
            self.draft = load_model(dcfg, self.device)
        if self.spec.method == "eagle3":
            from onecat_vllm.loader.weights import dummy_init, load_eagle3_weights, process_weights_after_loading
            from onecat_vllm.models.decoder import Eagle3Head
            dv = self.spec.draft_vocab_size
            if dv is None and self.spec.model and os.path.exists(os.path.join(self.spec.model, "config.json")):
                import json
                with open(os.path.join(self.spec.model, "config.json")) as f:
                    dv = json.load(f).get("draft_vocab_size")
            with torch.device(self.device):
                self.mtp = Eagle3Head(self.mc, self.model, self.device, dv)
            dummy_init(self.mtp, self.mc.seed + 1)
            if self.spec.model and os.path.isdir(self.spec.model):
                load_eagle3_weights(self.mtp, self.spec.model)
            process_weights_after_loading(self.mtp)
            self.mtp.eval()
            L = self.mc.num_hidden_layers
            aux = self.spec.eagle_aux_hidden_state_layers or (2, L // 2, L - 3)
            self.model.model.aux_hidden_layers = tuple(sorted(min(max(int(i), 0), L - 1) for i in aux))
            if len(set(self.model.model.aux_hidden_layers)) != 3:
                raise ValueError(f"EAGLE-3 needs three distinct target layers, got {aux} for a {L}-layer model")
        if self.spec.enabled:
            from onecat_vllm.spec_decode.proposers import make_proposer
            self.proposer = make_proposer(self)
        # user logits processors: ``module.path:ClassName`` (or dotted path), built once per worker as ``cls(vllm_config, device)``;
        # each step they get ``apply(logits [B, V] fp32, rows)`` with one dict per sampling request (reference: v1/sample/logits_processor/)
        self.custom_logits_processors = []
        for spec in self.mc.logits_processors or []:
            import importlib
            mod_name, _, cls_name = spec.replace(":", ".").rpartition(".")
            self.custom_logits_processors.append(getattr(importlib.import_module(mod_name), cls_name)(self.cfg, self.device))
        if self.mc.enable_lora:
            from onecat_vllm.lora import LoRAManager
            self.lora_manager = LoRAManager(self.model, self.mc.max_loras, self.mc.max_lora_rank, self.device, self.mc.dtype)
        log.info_once(f"model {self.mc.architecture} ready in {time.time() - t0:.1f}s on {self.device}")

    def get_kv_cache_specs(self) -> dict:
        mc, specs = self.mc, {}
        esz = torch.empty(0, dtype=self._kv_dtype()).element_size()
        asz = torch.empty(0, dtype=self._attn_kv_dtype()).element_size()
        for i, layer in self.model.model.local_layers():
            if layer.kind == "linear_attention":
                (cd, kw), (hv, k, v) = layer.linear_attn.state_shapes()
                nspec = self.num_spec + 1
                specs[f"layers.{i}"] = KVCacheSpec("mamba", self.block_size, 0, 0, 0,
                                                    state_bytes=(cd * kw * esz + hv * k * v * 4))
            elif layer.kind == "mla":
                specs[f"layers.{i}"] = KVCacheSpec("mla", self.block_size, 1, mc.kv_lora_rank + mc.qk_rope_head_dim, esz)
            else:
                specs[f"layers.{i}"] = KVCacheSpec("full", self.block_size, layer.self_attn.Hkv, mc.head_dim, asz)
        for i, layer in (self.draft.model.local_layers() if self.draft is not None else ()):
            specs[f"draft.{i}"] = KVCacheSpec("full", self.block_size, layer.self_attn.Hkv, self.draft.cfg.head_dim, asz)
        if self.mtp is not None:
            a = self.mtp.layer.self_attn
            if self.mc.use_mla:
                specs["mtp.0"] = KVCacheSpec("mla", self.block_size, 1, mc.kv_lora_rank + mc.qk_rope_head_dim, esz)
            else:
                specs["mtp.0"] = KVCacheSpec("full", self.block_size, a.Hkv, mc.head_dim, asz)
        return specs

    def _kv_dtype(self) -> torch.dtype:
        return self.mc.dtype

    def _attn_kv_dtype(self) -> torch.dtype:
        """Element type of the paged K/V of full-attention layers: ``--kv-cache-dtype fp8`` stores e4m3 bytes with unit scales
        (reference: config/cache.py ``cache_dtype``; csrc/cache_kernels.cu fp8 store). MLA latents and Gated-DeltaNet states keep
        the model dtype."""
        cd = self.cfg.cache_config.cache_dtype
        if cd in ("auto", "bfloat16", "bf16"):
            return self.mc.dtype
        if cd in ("fp8", "fp8_e4m3"):
            return torch.float8_e4m3fn
        raise ValueError(f"kv cache dtype {cd!r} is not supported (auto | fp8 | fp8_e4m3)")

    def zero_kv_cache(self) -> None:
        """After a sleep the cache pages are new physical memory: clear them (block 0 is the all-zero placeholder block)."""
        for c in list(self.kv_caches) + ([self.mtp_cache] if getattr(self, "mtp_cache", None) is not None else []):
            for t in (c if isinstance(c, tuple) else (c,)):
                if t is not None:
                    t.zero_()

    def initialize_kv_cache(self, kvc: KVCacheConfig) -> None:
        self.kv_cache_config = kvc
        dt, dev, nb, bs = self._kv_dtype(), self.device, kvc.num_blocks, self.block_size

        def alloc(spec: KVCacheSpec):
            if spec.kind == "mamba":
                return None
            if spec.kind == "mla":
                return torch.zeros(nb, bs, spec.head_size, dtype=dt, device=dev)
            return torch.zeros(nb, 2, spec.num_kv_heads, bs, spec.head_size, dtype=self._attn_kv_dtype(), device=dev)

        self.kv_caches = []
        for i, layer in self.model.model.local_layers():
            spec = kvc.layer_specs[f"layers.{i}"]
            if spec.kind == "mamba":
                (cd, kw), (hv, k, v) = layer.linear_attn.state_shapes()
                slots = kvc.num_state_slots
                self.kv_caches.append((torch.zeros(slots, cd, kw, dtype=dt, device=dev),
                                       torch.zeros(slots, hv, k, v, dtype=torch.float32, device=dev)))
            else:
                self.kv_caches.append(alloc(spec))
        if self.mtp is not None:
            self.mtp_cache = alloc(kvc.layer_specs["mtp.0"])
        if self.draft is not None:
            self.draft_caches = [alloc(kvc.layer_specs[f"draft.{i}"]) for i, _ in self.draft.model.local_layers()]
        # host mirror for the CPU tier of the prefix cache: same page layout, pinned when copies come from a GPU
        self.cpu_kv = []
        if kvc.num_cpu_blocks > 0:
            for c in self.kv_caches:
                m = torch.zeros((kvc.num_cpu_blocks,) + tuple(c.shape[1:]), dtype=c.dtype)
                self.cpu_kv.append(m.pin_memory() if self.use_cuda else m)
        self.max_blocks_per_req = -(-self.max_model_len // bs)
        self._init_buffers()

    def _init_buffers(self) -> None:
        """Pinned host staging + persistent device buffers (fixed addresses for CUDA graphs)."""
        T, R, MB = self.max_num_tokens, self.max_num_reqs, self.max_blocks_per_req
        pin = self.use_cuda

        def host(n, dt):
            t = torch.zeros(n, dtype=dt)
            return t.pin_memory() if pin else t

        # one packed int32 staging area: ids | positions | slot_mapping | qsl | seq_lens | state_slots | has_init | logit_idx
        # pdst | psrc: where last step's sampled tokens (still on the device) go in this step's ids (async scheduling)
        self._seg = {"ids": T, "pos": T, "slot": T, "qsl": R + 1, "seq": R, "sslot": R, "hinit": R, "lidx": T, "pdst": R, "psrc": R,
                     "pos3": 3 * T if getattr(self.mc, "mrope_section", None) else 0}  # [3, T] rotary positions (models with rotary sections)
        self._tcap = T
        total = sum(self._seg.values())
        self.h_pack = host(total, torch.int32)
        self.d_pack = torch.zeros(total, dtype=torch.int32, device=self.device)
        self.h_bt = host(R * MB, torch.int32).view(R, MB)
        self.d_bt = torch.zeros(R, MB, dtype=torch.int32, device=self.device)
        off, self._off = 0, {}
        for k, n in self._seg.items():
            self._off[k] = (off, n)
            off += n
        self.np_pack = self.h_pack.numpy()
        self.np_bt = self.h_bt.numpy()
        # per block-table row: the request state that owns it and how many of its blocks are already written there
        self._bt_owner, self._bt_written = [None] * self.np_bt.shape[0], [0] * self.np_bt.shape[0]
        # async scheduling: two pinned landing buffers for sampled tokens, the previous step's tokens on the device and which row
        # of them belongs to which request, the steps in flight, and an event after which the host staging may be rewritten
        self._tok_host = [host(T, torch.int64), host(T, torch.int64)]
        self._status_host = [host(16, torch.int32), host(16, torch.int32)]
        self._tok_flip = 0
        self._prev_toks, self._prev_row = None, {}
        self._inflight: list = []
        self._h2d_done = None
        self._n_patch = 0

    def _view(self, name: str, n: int, dev: bool = True) -> torch.Tensor:
        o, _ = self._off[name]
        return (self.d_pack if dev else self.h_pack)[o:o + n]

    # ------------------------------------------------------------------ state tracking
    def _update_states(self, so: SchedulerOutput) -> None:
        for rid in so.finished_req_ids:
            self.requests.pop(rid, None)
        # preempted requests stay known (sampling params, generator) until they resume or finish
        for nr in so.scheduled_new_reqs:
            sp = nr.sampling_params
            gen = None
            if sp is not None and sp.seed is not None:
                gen = torch.Generator(device=self.device)
                gen.manual_seed(sp.seed)
            self.requests[nr.req_id] = CachedRequestState(nr.req_id, list(nr.prompt_token_ids), len(nr.prompt_token_ids), sp,
                                                          list(nr.block_ids), nr.num_computed_tokens, nr.state_slot, gen, nr.eos_token_id,
                                                          nr.pooling_params, nr.lora_request,
                                                          nr.prompt_embeds.to(self.device, self.mc.dtype) if nr.prompt_embeds is not None else None,
                                                          list(nr.mm_features) if nr.mm_features else None)
        c = so.scheduled_cached_reqs
        for i, rid in enumerate(c.req_ids):
            st = self.requests.get(rid)
            if c.resumed_from_preemption[i] or st is None:
                toks = c.new_token_ids[i]
                old = st
                st = CachedRequestState(rid, list(toks), old.num_prompt_tokens if old else len(toks), old.sampling_params if old else None,
                                        list(c.new_block_ids[i] or []), c.num_computed_tokens[i], c.state_slots[i],
                                        old.generator if old else None, old.eos_token_id if old else None,
                                        old.pooling_params if old else None, old.lora_request if old else None,
                                        old.prompt_embeds if old else None, old.mm_features if old else None)
                self.requests[rid] = st
            else:
                st.num_computed_tokens = c.num_computed_tokens[i]
                if c.new_token_ids[i]:  # pipeline parallelism: tokens sampled on the last stage arrive through the scheduler
                    del st.token_ids[c.num_computed_tokens[i]:]
                    st.token_ids.extend(c.new_token_ids[i])
                if c.new_block_ids[i]:
                    st.block_ids.extend(c.new_block_ids[i])
                st.state_slot = c.state_slots[i]
                # the scheduler may have dropped tokens past a rejected draft; keep only what it counts

    # ------------------------------------------------------------------ input preparation
    def _prepare_inputs(self, so: SchedulerOutput):
        req_ids = list(so.num_scheduled_tokens.keys())
        R = len(req_ids)
        T = so.total_num_scheduled_tokens
        bs = self.block_size
        npk, o = self.np_pack, self._off
        ids = npk[o["ids"][0]: o["ids"][0] + T]
        pos = npk[o["pos"][0]: o["pos"][0] + T]
        slot = npk[o["slot"][0]: o["slot"][0] + T]
        qsl = npk[o["qsl"][0]: o["qsl"][0] + R + 1]
        seq = npk[o["seq"][0]: o["seq"][0] + R]
        sslot = npk[o["sslot"][0]: o["sslot"][0] + R]
        hinit = npk[o["hinit"][0]: o["hinit"][0] + R]
        lidx_buf = npk[o["lidx"][0]: o["lidx"][0] + self._seg["lidx"]]
        qsl[0] = 0
        t = 0
        max_q = max_s = 0
        logits_rows: list[int] = []  # how many logits rows each request contributes
        n_l = 0
        max_nb = 1
        drafts_of: list = []
        bt_owner, bt_written = self._bt_owner, self._bt_written
        pdst = npk[o["pdst"][0]: o["pdst"][0] + R]
        psrc = npk[o["psrc"][0]: o["psrc"][0] + R]
        n_patch = 0
        pos3 = npk[o["pos3"][0]: o["pos3"][0] + 3 * self._tcap].reshape(3, self._tcap) if self._seg["pos3"] else None
        if self._h2d_done is not None:
            self._h2d_done.synchronize()   # the previous step's copy out of this staging area has finished (it has, long ago)
        for r, rid in enumerate(req_ids):
            st = self.requests[rid]
            n = so.num_scheduled_tokens[rid]
            start = st.num_computed_tokens
            drafts = so.scheduled_spec_decode_tokens.get(rid, [])
            known = st.token_ids
            known_len = len(known) + st.pending
            end = start + n
            bl = st.block_ids
            nb = -(-end // bs)
            if st.pending and start == len(known):
                # the token at this position was sampled by the step in flight: it is patched in on the device
                assert n == 1 and rid in self._prev_row, "a pending token is the only input of its request"
                ids[t] = 0
                pos[t] = start
                slot[t] = bl[start // bs] * bs + start % bs
                pdst[n_patch], psrc[n_patch] = t, self._prev_row[rid]
                n_patch += 1
            elif n == 1 and start < len(known):
                # plain decode row: scalar writes, no temporaries
                ids[t] = known[start]
                pos[t] = start
                slot[t] = bl[start // bs] * bs + start % bs
            else:
                nk = min(end, len(known)) - start
                if nk > 0:
                    ids[t:t + nk] = known[start:start + nk]
                if end > len(known):
                    nd = end - len(known)
                    ids[t + nk:t + n] = drafts[:nd]
                pos[t:t + n] = np.arange(start, end, dtype=np.int32)
                b0 = start // bs
                b = np.asarray(bl[b0:nb], dtype=np.int32)
                p = pos[t:t + n]
                slot[t:t + n] = b[p // bs - b0] * bs + p % bs
            # block-table row: a request that kept its row only appends the blocks it gained (its list is append-only)
            if bt_owner[r] is st and bt_written[r] <= nb:
                w = bt_written[r]
                if w < nb:
                    self.np_bt[r, w:nb] = bl[w:nb]
            else:
                self.np_bt[r, :nb] = bl[:nb]
                bt_owner[r] = st
            bt_written[r] = nb
            max_nb = max(max_nb, nb)
            seq[r] = end
            sslot[r] = st.state_slot
            hinit[r] = 1 if start > 0 else 0
            # sampling positions: the request reaches the end of its known tokens in this step
            if end >= known_len:
                k = 1 + max(end - known_len, 0)
                lidx_buf[n_l:n_l + k] = np.arange(t + n - k, t + n, dtype=np.int32)
                n_l += k
                logits_rows.append(k)
            else:
                logits_rows.append(0)
            drafts_of.append(drafts[: max(end - known_len, 0)])
            if pos3 is not None:
                seg = pos[t:t + n]
                if st.mm_features and st.mrope is None:
                    from onecat_vllm.multimodal import mrope_positions
                    st.mrope, st.mrope_delta = mrope_positions(st.num_prompt_tokens, st.mm_features, getattr(self.mc, "vision_merge_size", 2))
                if st.mrope is None:
                    pos3[:, t:t + n] = seg
                else:
                    P = st.mrope.shape[1]
                    pos3[:, t:t + n] = np.where(seg < P, st.mrope[:, np.minimum(seg, P - 1)], seg + st.mrope_delta)
            t += n
            qsl[r + 1] = t
            max_q, max_s = max(max_q, n), max(max_s, end)
        assert t == T
        self._n_patch = n_patch
        return req_ids, R, T, n_l, logits_rows, drafts_of, max_q, max_s, max_nb

    def _pad_inputs(self, R: int, T: int, rp: int, q: int) -> None:
        """Fill the host staging arrays up to the captured batch size: padded requests own no tokens, padded tokens
        write no KV (slot -1)."""
        npk, o = self.np_pack, self._off
        tp = rp * q
        npk[o["ids"][0] + T: o["ids"][0] + tp] = 0
        npk[o["pos"][0] + T: o["pos"][0] + tp] = 0
        if self._seg["pos3"]:
            npk[o["pos3"][0]: o["pos3"][0] + 3 * self._tcap].reshape(3, self._tcap)[:, T:tp] = 0
        npk[o["slot"][0] + T: o["slot"][0] + tp] = -1
        npk[o["qsl"][0] + R + 1: o["qsl"][0] + rp + 1] = T
        npk[o["seq"][0] + R: o["seq"][0] + rp] = 0
        npk[o["sslot"][0] + R: o["sslot"][0] + rp] = 0
        npk[o["hinit"][0] + R: o["hinit"][0] + rp] = 0
        self.np_bt[R:rp, :1] = 0
        for r in range(R, rp):
            self._bt_owner[r] = None

    def _commit_inputs(self, R: int, T: int, n_l: int, max_nb: int) -> None:
        """Host → device copies of this step's inputs (non-blocking from pinned memory on GPUs)."""
        if self.use_cuda:
            self.d_pack.copy_(self.h_pack, non_blocking=True)
            self.d_bt[:R, :max_nb].copy_(self.h_bt[:R, :max_nb], non_blocking=True)
            self.h2d_bytes = self.h_pack.numel() * 4 + R * max_nb * 4
            if self._h2d_done is None:
                self._h2d_done = torch.cuda.Event()
            self._h2d_done.record()
        else:
            self.d_pack.copy_(self.h_pack)
            self.d_bt[:R, :max_nb].copy_(self.h_bt[:R, :max_nb])
        if self._n_patch:
            k = self._n_patch
            self._view("ids", T).index_copy_(0, self._view("pdst", k).long(), self._prev_toks[self._view("psrc", k).long()].to(torch.int32))

    def _build_metadata(self, R, T, max_q, max_s, max_nb, query_lens, seq_lens) -> AttentionMetadata:
        return AttentionMetadata(
            num_reqs=R, num_tokens=T, query_start_loc=self._view("qsl", R + 1), seq_lens=self._view("seq", R),
            block_table=self.d_bt[:R, :max_nb] if not self.use_cuda else self.d_bt[:R], slot_mapping=self._view("slot", T),
            positions=self._view("pos", T), max_query_len=max_q, max_seq_len=max_s, state_slots=self._view("sslot", R),
            has_initial_state=self._view("hinit", R), query_lens_cpu=query_lens, seq_lens_cpu=seq_lens,
            is_uniform_decode=(max_q == min(query_lens)) and max_q <= 1 + self.num_spec, uniform_query_len=max_q,
            mrope_positions=self._view("pos3", 3 * self._tcap).view(3, self._tcap)[:, :T] if self._seg["pos3"] else None)

    def _sampling_metadata(self, req_ids: list, rows: list[int]) -> SamplingMetadata:
        """One entry per *sampling request* (requests contributing logits rows this step)."""
        sel = [self.requests[rid] for rid, k in zip(req_ids, rows) if k > 0]
        sps = [s.sampling_params for s in sel]
        dev = self.device
        temps = [sp.temperature if sp else 0.0 for sp in sps]
        all_greedy = all(t < 1e-5 for t in temps)
        all_random = all(t >= 1e-5 for t in temps)
        # per-request sampling parameters travel through pinned memory: a copy from pageable memory would first wait for the
        # stream to drain, i.e. for a step that is still in flight
        def to_dev(xs, dt):
            t = torch.tensor(xs, dtype=dt)
            return t.pin_memory().to(dev, non_blocking=True) if self.use_cuda else t.to(dev)
        f32 = lambda xs: to_dev(xs, torch.float32)
        no_pen = all((sp is None) or (sp.presence_penalty == 0 and sp.frequency_penalty == 0 and sp.repetition_penalty == 1.0) for sp in sps)
        need_k = any(sp and sp.top_k > 0 for sp in sps)
        need_p = any(sp and sp.top_p < 1.0 for sp in sps)
        need_m = any(sp and sp.min_p > 0 for sp in sps)
        lps = [sp.logprobs for sp in sps if sp and sp.logprobs is not None]
        md = SamplingMetadata(
            temperature=None if all_greedy else f32(temps), all_greedy=all_greedy, all_random=all_random,
            top_p=f32([sp.top_p for sp in sps]) if need_p else None,
            top_k=to_dev([sp.top_k for sp in sps], torch.int64) if need_k else None,
            min_p=f32([sp.min_p for sp in sps]) if need_m else None,
            generators={i: s.generator for i, s in enumerate(sel) if s.generator is not None},
            max_num_logprobs=max(lps) if lps else None, no_penalties=no_pen)
        if not no_pen:
            md.presence_penalties = f32([sp.presence_penalty for sp in sps])
            md.frequency_penalties = f32([sp.frequency_penalty for sp in sps])
            md.repetition_penalties = f32([sp.repetition_penalty for sp in sps])
            md.prompt_token_ids = [s.token_ids[: s.num_prompt_tokens] for s in sel]
        md.output_token_ids = [s.token_ids[s.num_prompt_tokens:] for s in sel]
        for i, (s, sp) in enumerate(zip(sel, sps)):
            if sp is None:
                continue
            if sp.min_tokens > 0:
                stops = set(sp.all_stop_token_ids)
                if s.eos_token_id is not None and not sp.ignore_eos:
                    stops.add(s.eos_token_id)
                md.min_tokens[i] = (sp.min_tokens, stops)
            if sp.bad_words_token_ids:
                md.bad_words_token_ids[i] = sp.bad_words_token_ids
            if sp.thinking_token_budget is not None and sp._think_ids is not None:
                md.thinking[i] = (sp.thinking_token_budget, sp._think_ids[0], sp._think_ids[1])
        if self.custom_logits_processors:
            md.custom_processors = self.custom_logits_processors
            md.row_info = [dict(request_id=s.req_id, prompt_token_ids=s.token_ids[: s.num_prompt_tokens],
                                output_token_ids=s.token_ids[s.num_prompt_tokens:], extra_args=(sp.extra_args if sp else None) or {})
                           for s, sp in zip(sel, sps)]
        md.logit_bias = [sp.logit_bias if sp else None for sp in sps]
        md.allowed_token_ids = [sp.allowed_token_ids if sp else None for sp in sps]
        return md

    # ------------------------------------------------------------------ one step
    @torch.inference_mode()
    def _swap_kv(self, so: SchedulerOutput) -> None:
        """Copies of the CPU prefix-cache tier: evicted blocks to the host first, then restored blocks back
        (reference: v1/kv_offload/worker/cpu_gpu.py)."""
        if not (so.kv_swap_out or so.kv_swap_in):
            return
        if (so.kv_swap_out and isinstance(so.kv_swap_out[0][1], str)) or (so.kv_swap_in and isinstance(so.kv_swap_in[0][0], str)):
            return self._file_kv(so)
        if not self.cpu_kv:
            return
        if so.kv_swap_out:
            g = torch.tensor([a for a, _ in so.kv_swap_out], dtype=torch.long, device=self.device)
            c = torch.tensor([b for _, b in so.kv_swap_out], dtype=torch.long)
            for dev, host in zip(self.kv_caches, self.cpu_kv):
                host[c] = dev.index_select(0, g).cpu()
        if so.kv_swap_in:
            c = torch.tensor([a for a, _ in so.kv_swap_in], dtype=torch.long)
            g = torch.tensor([b for _, b in so.kv_swap_in], dtype=torch.long, device=self.device)
            for dev, host in zip(self.kv_caches, self.cpu_kv):
                dev.index_copy_(0, g, host[c].to(self.device, non_blocking=True))

    def _file_kv(self, so: SchedulerOutput) -> None:
        """Shared-storage connector: restores read ``[layers][page]`` tensors written by this or another engine. Saves are
        deferred until the step's forward has filled the blocks (``_save_kv_files``). Each rank writes its own shard."""
        from onecat_vllm.core import kv_p2p
        for f, g in so.kv_swap_in:
            if kv_p2p.is_p2p(f):
                host, port = self._p2p_endpoint()
                pages = kv_p2p.fetch_pages(host, port, f[len(kv_p2p.SCHEME):])
                if pages is None:
                    raise RuntimeError(f"the KV producer at {host}:{port} no longer holds block {f}")
            else:
                pages = torch.load(self._rank_file(f), map_location="cpu", weights_only=True)
            for dev, pg in zip(self.kv_caches, pages):
                dev[g].copy_(pg.to(self.device))
        self._pending_saves = list(so.kv_swap_out)

    def _rank_file(self, f: str) -> str:
        return f if self.pp.world_size == 1 else f"{f}.r{self.pp.rank}"

    def _p2p_endpoint(self) -> tuple:
        """This rank's end of the peer-to-peer KV connector: producer rank r listens on ``port + r``, consumer rank r asks there."""
        extra = (self.cfg.cache_config.kv_transfer_config or {}).get("kv_connector_extra_config") or {}
        return extra.get("host", "127.0.0.1"), int(extra.get("port", 14579)) + self.pp.rank

    def _save_kv_files(self) -> None:
        import os
        from onecat_vllm.core import kv_p2p
        for g, f in self._pending_saves:
            if kv_p2p.is_p2p(f):
                if getattr(self, "_kv_server", None) is None:
                    host, port = self._p2p_endpoint()
                    extra = (self.cfg.cache_config.kv_transfer_config or {}).get("kv_connector_extra_config") or {}
                    self._kv_server = kv_p2p.KVPageServer(host, port, int(extra.get("capacity_blocks", 4096)))
                self._kv_server.put(f[len(kv_p2p.SCHEME):], [dev[g].cpu() for dev in self.kv_caches])
                continue
            f = self._rank_file(f)
            tmp = f"{f}.tmp{os.getpid()}"
            torch.save([dev[g].cpu() for dev in self.kv_caches], tmp)
            os.replace(tmp, f)  # readers only ever see complete files
        self._pending_saves = []

    @torch.inference_mode()
    def execute_model(self, so: SchedulerOutput) -> ModelRunnerOutput:
        out = self._execute_model(so)
        if self._pending_saves:
            self._save_kv_files()
        return out

    # ---- async scheduling: a step is launched (inputs staged, forward and sampling enqueued, tokens on their way to pinned host
    # memory) and collected later, so the host work of the next step overlaps this one's device time. The engine only launches a
    # second step on top of one in flight when every request is plain (no penalties, logprobs, drafts, grammars): the unread tokens
    # are then needed nowhere but as the next step's input ids, where they are patched in on the device.
    # (reference: v1/core/sched/async_scheduler.py:12; v1/engine/core.py:568 ``step_with_batch_queue``;
    #  v1/worker/gpu_model_runner.py ``AsyncGPUModelRunnerOutput``)
    @torch.inference_mode()
    def launch_model(self, so: SchedulerOutput) -> None:
        res = self._execute_model(so, defer=True)
        self._inflight.append(res if isinstance(res, PendingStep) else PendingStep(out=res))

    @torch.inference_mode()
    def collect_model(self) -> ModelRunnerOutput:
        p = self._inflight.pop(0)
        out = p.out
        if p.done is not None:
            p.done.synchronize()
            host = p.host[:p.n].tolist()
            self.d2h_bytes = p.n * 8
            j = 0
            for i, k in enumerate(p.rows):
                if k > 0:
                    out.sampled_token_ids[i] = [host[j]]
                    st = self.requests.get(out.req_ids[i])
                    if st is not None:
                        st.token_ids.append(host[j])
                        st.pending = max(st.pending - 1, 0)
                    j += 1
            if p.ev is not None:
                out.device_time_ms = p.ev[0].elapsed_time(p.ev[1])
            if self.use_cuda and p.status is not None:
                st_word = 0
                for v in p.status.tolist():
                    st_word |= v
                out.status = st_word & 0xFFFFFFFF
        if self._pending_saves:
            self._save_kv_files()
        return out

    def _execute_model(self, so: SchedulerOutput, defer: bool = False):
        self._update_states(so)
        self._swap_kv(so)
        self._run_encoders(so)
        if so.total_num_scheduled_tokens == 0:
            return ModelRunnerOutput()
        req_ids, R, T, n_l, rows, drafts_of, max_q, max_s, max_nb = self._prepare_inputs(so)
        query_lens = [so.num_scheduled_tokens[r] for r in req_ids]
        seq_lens = [self.requests[r].num_computed_tokens + q for r, q in zip(req_ids, query_lens)]
        timed = self.use_cuda
        if timed:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        spec_any = any(len(d) > 0 for d in drafts_of)
        lora_batch = None
        if self.lora_manager is not None:
            from onecat_vllm.lora import set_active
            token_reqs = []
            for rid, qn in zip(req_ids, query_lens):
                token_reqs += [self.requests[rid].lora_request] * qn
            lora_batch = self.lora_manager.make_batch(token_reqs, self.device)
            set_active(lora_batch)
        gkey = None
        in_embed_prompt = any((self.requests[rid].prompt_embeds is not None or self.requests[rid].mm_features) and
                              self.requests[rid].num_computed_tokens < self.requests[rid].num_prompt_tokens for rid in req_ids)
        if self.graphs is not None and lora_batch is None and max_q == min(query_lens) and not (spec_any and self.mc.is_hybrid) and not in_embed_prompt:
            gkey = self.graphs.plan(R, max_q, max_s)
            if gkey is not None:
                self._pad_inputs(R, T, gkey[0], max_q)
        self._commit_inputs(max(R, gkey[0]) if gkey else R, T, n_l, max_nb)
        md = self._build_metadata(R, T, max_q, max_s, max_nb, query_lens, seq_lens)
        spec_verify = any(len(d) > 0 for d in drafts_of)
        gdn_spec = None
        if spec_verify and self.mc.is_hybrid:
            gdn_spec = md.gdn_record = []
            md.spec_q = 1 + self.num_spec
        ids = self._view("ids", T)
        hidden = None
        if gkey is not None:
            hidden = self.graphs.run(gkey, T)
        if hidden is None:
            inter = self._pp_recv(T) if not self.pp.is_first_pp else None
            hidden = self.model(ids, md, self.kv_caches, inputs_embeds=self._input_embeds(ids, req_ids, query_lens), intermediate=inter)
        if lora_batch is not None:
            from onecat_vllm.lora import set_active
            set_active(None)
        out = ModelRunnerOutput(req_ids=req_ids, sampled_token_ids=[[] for _ in req_ids])
        if not self.pp.is_last_pp:
            # hand (block output, residual) to the next stage; sampling happens on the last one
            self._pp_send(hidden)
            if timed:
                ev1.record()
                torch.cuda.synchronize()
                out.device_time_ms = ev0.elapsed_time(ev1)
            return out
        sampled_lists: list[list[int]] = [[] for _ in req_ids]
        if n_l > 0:
            lidx = self._view("lidx", n_l).long()
            sample_hidden = hidden[lidx]
            smd = self._sampling_metadata(req_ids, rows)
            toks = None
            if (self.pp.tp_size > 1 and not spec_verify and so.grammar_bitmask is None and smd.max_num_logprobs is None
                    and self.sampler.is_plain_greedy(smd)):
                # tensor-parallel greedy decoding: one (value, index) pair per row crosses the ranks instead of the vocabulary
                toks = self.model.greedy_tokens(sample_hidden)
            if toks is None:
                logits = self.model.compute_logits(sample_hidden)
            if so.grammar_bitmask is not None:
                smd.grammar_bitmask = self._grammar_mask(so, req_ids, rows, logits.shape[-1])
            samp_rows = [k for k in rows if k > 0]
            if not spec_verify:
                so_ = self.sampler(logits, smd) if toks is None else SamplerOutput(toks, None)
                toks = so_.sampled_token_ids
                if timed:
                    ev1.record()
                if defer and so_.logprobs is None and self.proposer is None:
                    # leave the tokens on the device for the next step's inputs and send a copy towards the host
                    buf, sbuf = self._tok_host[self._tok_flip], self._status_host[self._tok_flip]
                    self._tok_flip ^= 1
                    n_s = toks.shape[0]
                    buf[:n_s].copy_(toks, non_blocking=True)
                    done = None
                    if self.use_cuda:
                        from onecat_vllm.ops import _C
                        _C.read_status_async(sbuf)   # the kernels' status words ride along: no device-wide wait when they are read
                        done = torch.cuda.Event()
                        done.record()
                    self._prev_toks, self._prev_row = toks, {}
                    j = 0
                    for i, k in enumerate(rows):
                        if k > 0:
                            self._prev_row[req_ids[i]] = j
                            self.requests[req_ids[i]].pending += 1
                            j += 1
                    return PendingStep(out, rows, n_s, buf, done if done is not None else _Ready(), (ev0, ev1) if timed else None, sbuf)
                host = toks.tolist()  # device → host read of the step's result
                self.d2h_bytes = len(host) * 8
                j = 0
                for i, k in enumerate(rows):
                    if k > 0:
                        sampled_lists[i] = [host[j]]
                        j += 1
                out.logprobs = self._scatter_logprobs(so_.logprobs, rows)
            else:
                sampled_lists = self._verify(logits, smd, rows, drafts_of)
                if timed:
                    ev1.record()
        elif timed:
            ev1.record()
        out.prompt_logprobs = self._prompt_logprobs(hidden, req_ids, query_lens)
        if any(self.requests[r].pooling_params is not None for r in req_ids):
            out.pooler_output = self._pool(hidden, req_ids, query_lens, rows)
        if gdn_spec:
            self._commit_gdn_spec(gdn_spec, md, sampled_lists, query_lens)
        # bookkeeping: the runner owns the token history of running requests
        for i, rid in enumerate(req_ids):
            st = self.requests[rid]
            if sampled_lists[i]:
                end = st.num_computed_tokens + query_lens[i]
                # tokens are appended after the last *known* token
                st.token_ids.extend(sampled_lists[i])
        out.sampled_token_ids = sampled_lists
        if self.proposer is not None and n_l > 0:
            out.spec_token_ids = self.proposer.propose(self, so, req_ids, rows, sampled_lists, hidden, md, drafts_of)
        if timed:
            torch.cuda.synchronize()
            out.device_time_ms = ev0.elapsed_time(ev1)
        if self.use_cuda:
            from onecat_vllm.ops import cuda as K
            out.status = K.check_status()
        return out

    def _prompt_logprobs(self, hidden: torch.Tensor, req_ids: list, query_lens: list[int]):
        """Log-probabilities of the prompt tokens that this step's chunk predicts, for requests that asked for them: per request a
        list of (token ids, logprobs, rank) with the actual next prompt token first and then the top-k (reference:
        v1/worker/gpu_model_runner.py ``_get_prompt_logprobs_dict``). Rows are scored in slices to bound the logits buffer."""
        res, o = None, 0
        for rid, q in zip(req_ids, query_lens):
            st = self.requests[rid]
            sp = st.sampling_params
            k = sp.prompt_logprobs if sp is not None else None
            c0 = st.num_computed_tokens
            if k is not None and c0 < st.num_prompt_tokens - 1:
                n = min(c0 + q, st.num_prompt_tokens - 1) - c0  # rows whose next token is still a prompt token
                tgt = torch.tensor(st.token_ids[c0 + 1:c0 + 1 + n], dtype=torch.long, device=self.device)
                ids, lps, ranks = [], [], []
                for a in range(0, n, 512):
                    b = min(a + 512, n)
                    lp = torch.log_softmax(self.model.compute_logits(hidden[o + a:o + b]).float(), dim=-1)
                    i_, v_, r_ = Sampler.gather_logprobs(lp, k, tgt[a:b])
                    ids += i_.tolist()
                    lps += v_.tolist()
                    ranks += r_.tolist()
                res = res or {}
                res[rid] = [(ids[j], lps[j], ranks[j]) for j in range(n)]
            o += q
        return res

    def _run_encoders(self, so) -> None:
        """Encode the multimodal items the scheduler put into this step and drop the outputs it released
        (reference: v1/worker/gpu_model_runner.py ``_execute_mm_encoder``; encoder cache keyed by the item's content hash)."""
        for h in getattr(so, "free_encoder_mm_hashes", None) or ():
            self.encoder_cache.pop(h, None)
        for rid, idxs in (getattr(so, "scheduled_encoder_inputs", None) or {}).items():
            st = self.requests[rid]
            for i in idxs:
                f = st.mm_features[i]
                if f.mm_hash in self.encoder_cache:
                    continue
                out = self.model.embed_multimodal(f, self.device)
                if out.shape[0] != f.length or out.shape[1] != self.mc.hidden_size:
                    raise ValueError(f"the encoder returned {tuple(out.shape)} for an item of {f.length} positions")
                self.encoder_cache[f.mm_hash] = out.to(self.device, self.mc.dtype)

    def _input_embeds(self, ids: torch.Tensor, req_ids: list, query_lens: list[int]) -> Optional[torch.Tensor]:
        """Embedding rows of the step with the prompt positions of ``prompt_embeds`` requests replaced by their own vectors and the
        placeholder positions of multimodal items by their encoder outputs; ``None`` when no such position is in the batch
        (reference: v1/worker/gpu_model_runner.py ``enable_prompt_embeds`` path and ``_gather_mm_embeddings``)."""
        if not self.pp.is_first_pp:
            return None
        emb, o = None, 0
        for rid, q in zip(req_ids, query_lens):
            st = self.requests[rid]
            c0 = st.num_computed_tokens
            if st.prompt_embeds is not None and c0 < st.num_prompt_tokens:
                if emb is None:
                    emb = self.model.model.embed_tokens(ids)
                n = min(q, st.num_prompt_tokens - c0)
                emb[o:o + n] = st.prompt_embeds[c0:c0 + n]
            for f in st.mm_features or ():
                lo, hi = max(f.offset, c0), min(f.offset + f.length, c0 + q)
                if lo >= hi:
                    continue
                if emb is None:
                    emb = self.model.model.embed_tokens(ids)
                emb[o + lo - c0: o + hi - c0] = self.encoder_cache[f.mm_hash][lo - f.offset: hi - f.offset]
            o += q
        return emb

    def _pool(self, hidden: torch.Tensor, req_ids: list, query_lens: list[int], rows: list[int]) -> list:
        """Pooled final-norm hidden state of embedding requests: last token, first token or mean over the prompt (accumulated
        across prefill chunks), L2-normalised on request (reference: model_executor/layers/pooler/ ``LastPool``/``MeanPool``/
        ``CLSPool`` + ``PoolerNormalize``; v1/pool/metadata.py)."""
        out: list = [None] * len(req_ids)
        o = 0
        for i, (rid, q) in enumerate(zip(req_ids, query_lens)):
            st = self.requests[rid]
            pp = st.pooling_params
            if pp is not None:
                h = hidden[o:o + q].float()
                if pp.pooling_type == "mean":
                    s = h.sum(0)
                    st.pool_sum = s if st.pool_sum is None else st.pool_sum + s
                elif pp.pooling_type == "cls" and st.num_computed_tokens == 0:
                    st.pool_first = h[0].clone()
                if rows[i] > 0:  # the prompt is complete in this step
                    n_prompt = st.num_computed_tokens + q
                    v = h[-1] if pp.pooling_type == "last" else (st.pool_sum / n_prompt if pp.pooling_type == "mean" else st.pool_first)
                    if pp.task == "classify":
                        head = getattr(self.model, "score", None)
                        if head is None:
                            raise ValueError("classify needs a *ForSequenceClassification checkpoint")
                        v = head(v.to(self.mc.dtype).unsqueeze(0))[0].float()
                        if pp.use_activation:
                            v = torch.sigmoid(v) if v.numel() == 1 else torch.softmax(v, -1)
                        out[i] = v.cpu().tolist()
                        o += q
                        continue
                    if pp.dimensions:
                        v = v[: pp.dimensions]
                    if pp.normalize:
                        v = v / v.norm().clamp_min(1e-12)
                    out[i] = v.cpu().tolist()
            o += q
        return out

    # ---- pipeline parallelism: stage boundaries carry two [T, hidden] tensors (reference: gpu_worker.py:80-110, 792-880
    # ``IntermediateTensors`` send/recv; v1/worker/gpu_model_runner.py:8437-8443)
    def _pp_send(self, pair) -> None:
        import torch.distributed as dist
        dst = ps.pp_neighbor(+1)
        for t in pair:
            dist.send(t.contiguous(), dst=dst)

    def _pp_recv(self, T: int) -> tuple:
        import torch.distributed as dist
        src = ps.pp_neighbor(-1)
        out = []
        for _ in range(2):
            t = torch.empty(T, self.mc.hidden_size, dtype=self.mc.dtype, device=self.device)
            dist.recv(t, src=src)
            out.append(t)
        return tuple(out)

    def _grammar_mask(self, so: SchedulerOutput, req_ids: list, rows: list[int], vocab: int) -> torch.Tensor:
        """Packed per-request words → bool ``[sampling requests, vocab]`` (True = allowed); requests without a grammar get
        all-ones rows. Requests under a grammar never carry drafts, so their single logits row is the one the sampler
        sees (reference: v1/structured_output/utils.py ``apply_grammar_bitmask``)."""
        import numpy as np
        n = sum(1 for k in rows if k > 0)
        packed = np.full((n, so.grammar_bitmask.shape[1]), -1, dtype=np.int32)
        o = 0
        for rid, k in zip(req_ids, rows):
            if k == 0:
                continue
            r = so.structured_rows.get(rid)
            if r is not None:
                packed[o] = so.grammar_bitmask[r]
            o += 1
        words = torch.from_numpy(packed).to(self.device, non_blocking=True)
        shifts = torch.arange(32, device=self.device, dtype=torch.int32)
        bits = ((words.unsqueeze(-1) >> shifts) & 1).bool().reshape(words.shape[0], -1)
        if bits.shape[1] < vocab:  # logits rows padded beyond the tokenizer's vocabulary stay masked out
            bits = torch.nn.functional.pad(bits, (0, vocab - bits.shape[1]), value=False)
        return bits[:, :vocab]

    def _scatter_logprobs(self, lp, rows):
        if lp is None:
            return None
        lists = to_logprobs_lists(lp, [1] * sum(1 for k in rows if k > 0))
        out, j = [], 0
        for k in rows:
            if k > 0:
                out.append(lists[j])
                j += 1
            else:
                out.append(None)
        return out

    @staticmethod
    def _verify_is_unconstrained(md: SamplingMetadata) -> bool:
        """No request asks for anything that changes the target distribution beyond the temperature."""
        return (md.no_penalties and md.top_k is None and md.top_p is None and md.min_p is None and not md.min_tokens and
                not any(md.logit_bias) and not any(a is not None for a in md.allowed_token_ids) and not md.bad_words_token_ids and
                not md.thinking and not md.custom_processors)

    def _expand_sampling_metadata(self, md: SamplingMetadata, drafts: list):
        """Sampling state with one row per verified draft position (request b contributes ``len(drafts[b])`` rows; row i sees the
        request's output followed by its first i drafts), the owner of every row, and the state of the bonus rows (one per request,
        whose context includes all of its drafts). The grammar bitmask stays with the bonus rows."""
        owner = [b for b, d in enumerate(drafts) for _ in d]
        dev = self.device
        idx = torch.tensor(owner, dtype=torch.long, device=dev)
        pick = lambda t: t.index_select(0, idx) if t is not None else None
        ctx = [md.output_token_ids[b] + list(d[:i]) for b, d in enumerate(drafts) for i in range(len(d))]
        emd = SamplingMetadata(
            temperature=pick(md.temperature), all_greedy=md.all_greedy, all_random=md.all_random, top_p=pick(md.top_p), top_k=pick(md.top_k),
            min_p=pick(md.min_p), generators={}, max_num_logprobs=None, no_penalties=md.no_penalties,
            presence_penalties=pick(md.presence_penalties), frequency_penalties=pick(md.frequency_penalties),
            repetition_penalties=pick(md.repetition_penalties),
            prompt_token_ids=[md.prompt_token_ids[b] for b in owner] if md.prompt_token_ids else None, output_token_ids=ctx,
            min_tokens={r: md.min_tokens[b] for r, b in enumerate(owner) if b in md.min_tokens},
            logit_bias=[md.logit_bias[b] for b in owner] if md.logit_bias else [],
            allowed_token_ids=[md.allowed_token_ids[b] for b in owner] if md.allowed_token_ids else [],
            bad_words_token_ids={r: md.bad_words_token_ids[b] for r, b in enumerate(owner) if b in md.bad_words_token_ids},
            thinking={r: md.thinking[b] for r, b in enumerate(owner) if b in md.thinking}, custom_processors=md.custom_processors,
            row_info=[dict(md.row_info[b], output_token_ids=ctx[r]) for r, b in enumerate(owner)] if md.row_info else [])
        import dataclasses
        full = [md.output_token_ids[b] + list(d) for b, d in enumerate(drafts)]
        bonus = dataclasses.replace(md, output_token_ids=full,
                                    row_info=[dict(ri, output_token_ids=full[b]) for b, ri in enumerate(md.row_info)] if md.row_info else [])
        return emd, owner, bonus

    def _verify(self, logits, smd, rows, drafts_of) -> list[list[int]]:
        """Rejection-sample requests that carried drafts; plain-sample the rest. ``logits`` rows are grouped per
        request (k_i + 1 rows for a request with k_i drafts)."""
        k = self.num_spec
        B = sum(1 for r in rows if r > 0)
        V = logits.shape[-1]
        dev = logits.device
        live = [(r, drafts_of[i]) for i, r in enumerate(rows) if r > 0]
        if live and all(r == k + 1 and len(d) == k for r, d in live) and logits.is_contiguous() and logits.shape[0] == B * (k + 1):
            # every request verified a full set of drafts (the steady state of decoding): the logits already are [B, k + 1, V]
            tl = logits.view(B, k + 1, V)
            if not self._verify_is_unconstrained(smd):
                tl = tl.clone()      # constrained rows are rewritten below; the caller's logits stay as they are
            draft = torch.tensor([d for _, d in live], dtype=torch.long).to(dev)
            nd = torch.full((B,), k, dtype=torch.long, device=dev)
            last_rows = [b * (k + 1) + k for b in range(B)]
        else:
            tl = torch.zeros(B, k + 1, V, dtype=logits.dtype, device=dev)
            draft = torch.zeros(B, k, dtype=torch.long, device=dev)
            nd = torch.zeros(B, dtype=torch.long, device=dev)
            last_rows, j, b = [], 0, 0
            nd_host = []
            for i, r in enumerate(rows):
                if r == 0:
                    continue
                d = drafts_of[i]
                tl[b, :r] = logits[j:j + r]
                if d:
                    draft[b, : len(d)] = torch.tensor(d, device=dev)
                nd_host.append(len(d))
                last_rows.append(j + r - 1)
                j += r
                b += 1
            nd.copy_(torch.tensor(nd_host))
        bonus_md = smd
        if not self._verify_is_unconstrained(smd):
            # The drafts are judged against the distribution the sampler would have drawn from: every verified row goes through the
            # logit processors and penalties (its context being the request's output plus the drafts before it) and the top-k /
            # top-p / min-p filters, exactly as the bonus row does
            # (reference: v1/sample/rejection_sampler.py ``apply_logits_processors`` / ``apply_sampling_constraints``).
            kept = [d for i, d in enumerate(drafts_of) if rows[i] > 0]
            emd, owner, bonus_md = self._expand_sampling_metadata(smd, kept)
            flat = torch.cat([tl[b, :len(d)] for b, d in enumerate(kept) if d]).float() if any(kept) else None
            if flat is not None:
                flat = Sampler.apply_logits_processors(flat, emd)
                flat = Sampler.apply_penalties(flat, emd)
                for proc in emd.custom_processors:
                    flat = proc.apply(flat, emd.row_info)
                if emd.top_k is not None or emd.top_p is not None or emd.min_p is not None:
                    t = emd.temperature if emd.temperature is not None else torch.ones(flat.shape[0], device=dev)
                    t = torch.where(t < 1e-5, torch.ones_like(t), t).unsqueeze(-1)
                    flat = ref_ops.top_k_top_p_min_p(flat / t, emd.top_k, emd.top_p, emd.min_p) * t   # masked entries stay -inf
                j = 0
                for b, d in enumerate(kept):
                    if d:
                        tl[b, :len(d)] = flat[j:j + len(d)].to(tl.dtype)
                        j += len(d)
        bonus = self.sampler(logits[torch.tensor(last_rows, device=dev)], bonus_md).sampled_token_ids
        res = self.rejection_sampler(draft, nd, tl, bonus, smd)
        parsed = RejectionSampler.parse_output(res)
        self.d2h_bytes = res.numel() * 8
        out, b = [], 0
        for r in rows:
            if r == 0:
                out.append([])
            else:
                out.append(parsed[b])
                b += 1
        return out

    # ---- Gated-DeltaNet state under speculation: the forward records the state after every verified token; once the
    # accepted count is known each layer's slot takes the state that follows the last accepted token
    def _commit_gdn_spec(self, rec: list, md, sampled, query_lens) -> None:
        n_valid = torch.tensor([len(s) if s else q for s, q in zip(sampled, query_lens)], dtype=torch.int32, device=self.device)
        if self.use_cuda:
            from onecat_vllm.ops import cuda as K
            K.gdn_commit(md, rec, n_valid)
            return
        from onecat_vllm.ops import ref
        qsl = md.query_start_loc.tolist()
        slots = md.state_slots.tolist()
        for e in rec:
            for r in range(md.num_reqs):
                a, b = qsl[r], qsl[r + 1]
                n = int(n_valid[r])
                if b - a <= e["spec"].shape[1]:
                    e["ssm_state"][slots[r]] = e["spec"][r, min(n, b - a) - 1]
                e["conv_state"][slots[r]] = ref.conv_state_after(e["prev"][r], e["mixed"][a:b], n)

    # ------------------------------------------------------------------ profiling helpers
    @torch.inference_mode()
    def dummy_run(self, num_tokens: int, num_reqs: int = 1) -> None:
        """Max-shape forward used for memory profiling and kernel warm-up; touches no request state."""
        T, R = num_tokens, max(1, min(num_reqs, num_tokens))
        per = T // R
        qsl = torch.arange(0, R + 1, dtype=torch.int32, device=self.device) * per
        qsl[-1] = T
        seq = (qsl[1:] - qsl[:-1]).to(torch.int32)
        nb = -(-int(seq.max()) // self.block_size)
        md = AttentionMetadata(R, T, qsl, seq, torch.zeros(R, max(nb, 1), dtype=torch.int32, device=self.device),
                               torch.full((T,), -1, dtype=torch.int32, device=self.device),
                               torch.zeros(T, dtype=torch.int32, device=self.device), int(seq.max()), int(seq.max()),
                               torch.zeros(R, dtype=torch.int32, device=self.device), torch.zeros(R, dtype=torch.int32, device=self.device),
                               seq.tolist(), seq.tolist())
        ids = torch.zeros(T, dtype=torch.int32, device=self.device)
        caches = self.kv_caches if self.kv_caches else self._tiny_caches()
        inter = None
        if not self.pp.is_first_pp:  # profiling never communicates: each stage runs on zeros
            inter = (torch.zeros(T, self.mc.hidden_size, dtype=self.mc.dtype, device=self.device),) * 2
        h = self.model(ids, md, caches, intermediate=inter)
        if self.pp.is_last_pp:
            self.model.compute_logits(h[:R])

    def _tiny_caches(self):
        """One-block caches so the profiling forward can run before the real cache exists."""
        out = []
        dt = self._kv_dtype()
        for _, layer in self.model.model.local_layers():
            if layer.kind == "linear_attention":
                (cd, kw), (hv, k, v) = layer.linear_attn.state_shapes()
                out.append((torch.zeros(1, cd, kw, dtype=dt, device=self.device), torch.zeros(1, hv, k, v, dtype=torch.float32, device=self.device)))
            elif layer.kind == "mla":
                out.append(torch.zeros(1, self.block_size, self.mc.kv_lora_rank + self.mc.qk_rope_head_dim, dtype=dt, device=self.device))
            else:
                out.append(torch.zeros(1, 2, layer.self_attn.Hkv, self.block_size, self.mc.head_dim, dtype=dt, device=self.device))
        return out
