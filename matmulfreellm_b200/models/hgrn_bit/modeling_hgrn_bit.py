"""HGRNBit model classes with the reference's names, constructor arguments, parameter names and forward
signatures (mmfreelm/models/hgrn_bit/modeling_hgrn_bit.py), inference only."""
from __future__ import annotations

import math
import warnings
from typing import List, Optional, Tuple, Union

import torch
import torch.nn as nn
from transformers.modeling_outputs import BaseModelOutputWithPast, CausalLMOutputWithPast
from transformers.modeling_utils import PreTrainedModel

from ... import kernels
from ...layers.hgrn_bit import HGRNBitAttention
from ...modules import RMSNorm
from ...modules.activations import swiglu
from ...ops.fusedbitnet import BitLinear as _BitLinearBase
from ...ops.fusedbitnet import FusedBitLinear as BitLinear
from ..utils import RecurrentCache
from .configuration_hgrn_bit import HGRNBitConfig


class HGRNBitMLP(nn.Module):
    """down_proj(silu(gate) * y) with (gate, y) = gate_proj(x).chunk(2, -1)  (modeling_hgrn_bit.py:29-59)."""

    def __init__(self, hidden_size: int, hidden_ratio: Optional[int] = None, intermediate_size: Optional[int] = None,
                 hidden_act: str = "swish"):
        super().__init__()
        self.hidden_size = hidden_size
        hidden_ratio = 4 if hidden_ratio is None else hidden_ratio
        if intermediate_size is None:  # multiple of 256 at or above 2/3 * hidden_ratio * hidden_size
            intermediate_size = 256 * ((int(hidden_size * hidden_ratio * 2 / 3) + 255) // 256)
        if hidden_act not in ("swish", "silu"):
            raise NotImplementedError("the MLP is SiLU-gated (hidden_act 'swish')")
        self.hidden_ratio, self.intermediate_size = hidden_ratio, intermediate_size
        self.gate_proj = BitLinear(hidden_size, intermediate_size * 2, bias=False)
        self.down_proj = BitLinear(intermediate_size, hidden_size, bias=False)

    def forward(self, x):
        gate, y = self.gate_proj(x).chunk(2, -1)
        return self.down_proj(swiglu(gate, y))


class HGRNBitBlock(nn.Module):
    def __init__(self, config: HGRNBitConfig, layer_idx: int):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.attn_norm = RMSNorm(hidden_size=config.hidden_size, eps=config.rms_norm_eps)
        self.attn = HGRNBitAttention(mode=config.attn_mode, hidden_size=config.hidden_size,
                                     num_heads=config.num_heads, expand_ratio=config.expand_ratio,
                                     use_short_conv=config.use_short_conv, conv_size=config.conv_size,
                                     share_conv_kernel=config.share_conv_kernel, layernorm_eps=config.rms_norm_eps,
                                     layer_idx=layer_idx)
        self.mlp_norm = RMSNorm(hidden_size=config.hidden_size, eps=config.rms_norm_eps)
        self.mlp = HGRNBitMLP(hidden_size=config.hidden_size, hidden_ratio=config.hidden_ratio,
                              intermediate_size=config.intermediate_size, hidden_act=config.hidden_act)

    def forward(self, hidden_states, attention_mask=None, past_key_values=None, use_cache=False,
                output_attentions=False, lower_bound=False, **kwargs):
        residual = hidden_states
        hidden_states = self.attn_norm(hidden_states)
        hidden_states, attentions, past_key_values = self.attn(
            hidden_states=hidden_states, attention_mask=attention_mask, past_key_values=past_key_values,
            use_cache=use_cache, output_attentions=output_attentions, lower_bound=lower_bound)
        hidden_states, residual = self.mlp_norm(hidden_states, residual, True)
        hidden_states = residual + self.mlp(hidden_states)
        return hidden_states, attentions, past_key_values


class HGRNBitPreTrainedModel(PreTrainedModel):
    config_class = HGRNBitConfig
    supports_gradient_checkpointing = False
    _no_split_modules = ["HGRNBitBlock"]

    def _init_weights(self, module: nn.Module, rescale_prenorm_residual: bool = True,
                      num_residuals_per_layer: int = 2):
        std = self.config.initializer_range
        if isinstance(module, (nn.Linear, nn.Conv1d)):
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=std)
            if module.padding_idx is not None:
                module.weight.data[module.padding_idx].zero_()
        if rescale_prenorm_residual:  # 1/sqrt(2L) on the two residual-writing projections (:142-156)
            for name, p in module.named_parameters():
                # a parameter that from_pretrained has just loaded is marked by transformers and must not be rescaled
                # again (the wrapped nn.init functions above honour the mark by themselves; this in-place division does not)
                if name in ("o_proj.weight", "down_proj.weight") and not getattr(p, "_is_hf_initialized", False):
                    with torch.no_grad():
                        p /= math.sqrt(num_residuals_per_layer * self.config.num_hidden_layers)

    def pack_weights(self):
        """Ternarise and 2-bit pack every BitLinear from its current latent weight (the offline step).
        Call while the weights are still fp32, i.e. before `.half()` / `.bfloat16()`."""
        for m in self.modules():
            if isinstance(m, _BitLinearBase):
                m.pack_weights()
        return self


class HGRNBitModel(HGRNBitPreTrainedModel):
    def __init__(self, config: HGRNBitConfig):
        super().__init__(config)
        self.padding_idx = config.pad_token_id
        self.vocab_size = config.vocab_size
        self.embeddings = nn.Embedding(config.vocab_size, config.hidden_size, self.padding_idx)
        if config.use_lower_bound:
            self.lower_bounds = nn.Parameter(torch.zeros(config.num_hidden_layers, config.hidden_size))
        self.layers = nn.ModuleList([HGRNBitBlock(config, i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)
        self.gradient_checkpointing = False
        self.post_init()

    def get_input_embeddings(self):
        return self.embeddings

    def set_input_embeddings(self, value):
        self.embeddings = value

    def layer_lower_bounds(self) -> Optional[torch.Tensor]:
        """[L, hidden] cumulative-softmax lower bounds of the forget gates (:231-233); row 0 is unused."""
        if not self.config.use_lower_bound:
            return None
        lb = self.lower_bounds.softmax(0)
        return lb.cumsum(0) - lb[0]

    def forward(self, input_ids: Optional[torch.LongTensor] = None, attention_mask: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.FloatTensor] = None, past_key_values=None,
                use_cache: Optional[bool] = None, output_attentions: Optional[bool] = None,
                output_hidden_states: Optional[bool] = None, return_dict: Optional[bool] = None
                ) -> Union[Tuple, BaseModelOutputWithPast]:
        if output_attentions:
            warnings.warn("`HGRNBitModel` does not `output_attentions` now, setting it to `False`.")
        output_attentions = False
        if output_hidden_states is None:
            output_hidden_states = bool(getattr(self.config, "output_hidden_states", False))
        if use_cache is None:
            use_cache = self.config.use_cache if not self.training else False
        if return_dict is None:
            return_dict = bool(getattr(self.config, "return_dict", True))
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("You cannot specify both input_ids and inputs_embeds at the same time")
        if input_ids is None and inputs_embeds is None:
            raise ValueError("You have to specify either input_ids or inputs_embeds")
        batch_size = input_ids.shape[0] if input_ids is not None else inputs_embeds.shape[0]

        if inputs_embeds is None:
            inputs_embeds = kernels.embedding(self.embeddings.weight, input_ids)
        hidden_states = inputs_embeds

        if use_cache:
            if past_key_values is None:
                past_key_values = [layer.attn.init_state(batch_size) for layer in self.layers]
            if not isinstance(past_key_values, RecurrentCache):
                past_key_values = RecurrentCache.from_legacy_cache(past_key_values)

        all_hidden_states = () if output_hidden_states else None
        lower_bounds = self.layer_lower_bounds()
        for i, layer in enumerate(self.layers):
            if output_hidden_states:
                all_hidden_states += (hidden_states,)
            hidden_states, _, past_key_values = layer(
                hidden_states, attention_mask=attention_mask, past_key_values=past_key_values, use_cache=use_cache,
                output_attentions=False, lower_bound=None if lower_bounds is None else lower_bounds[i])
        hidden_states = self.norm(hidden_states)
        if output_hidden_states:
            all_hidden_states += (hidden_states,)

        next_cache = past_key_values.to_legacy_cache() if use_cache else None
        if not return_dict:
            return tuple(x for x in (hidden_states, next_cache, all_hidden_states) if x is not None)
        return BaseModelOutputWithPast(last_hidden_state=hidden_states, past_key_values=next_cache,
                                       hidden_states=all_hidden_states, attentions=None)


class HGRNBitForCausalLM(HGRNBitPreTrainedModel):
    # transformers >= 5 wants {tied parameter: its source}; only used when config.tie_word_embeddings is set
    _tied_weights_keys = {"lm_head.weight": "model.embeddings.weight"}

    def __init__(self, config):
        super().__init__(config)
        self.model = HGRNBitModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = BitLinear(config.hidden_size, config.vocab_size, bias=False)
        self.post_init()

    def get_input_embeddings(self):
        return self.model.embeddings

    def set_input_embeddings(self, value):
        self.model.embeddings = value

    def get_output_embeddings(self):
        return self.lm_head

    def set_output_embeddings(self, new_embeddings):
        self.lm_head = new_embeddings

    def set_decoder(self, decoder):
        self.model = decoder

    def get_decoder(self):
        return self.model

    def prepare_inputs_for_generation(self, input_ids: torch.LongTensor = None, past_key_values=None,
                                      attention_mask: Optional[torch.Tensor] = None,
                                      inputs_embeds: Optional[torch.Tensor] = None, **kwargs):
        if past_key_values is not None:   # with a cache only the newest token is fed (:335-338)
            if not isinstance(past_key_values, RecurrentCache):
                past_key_values = RecurrentCache.from_legacy_cache(past_key_values, input_ids.shape[1] - 1)
            input_ids = input_ids[:, -1:]
            if attention_mask is not None:
                attention_mask = attention_mask[:, -1:]
        if inputs_embeds is not None and past_key_values is None:
            model_inputs = {"inputs_embeds": inputs_embeds}
        else:
            model_inputs = {"input_ids": input_ids.contiguous()}
        model_inputs.update({"past_key_values": past_key_values, "use_cache": kwargs.get("use_cache"),
                             "attention_mask": attention_mask})
        return model_inputs

    def forward(self, input_ids: torch.LongTensor = None, attention_mask: Optional[torch.Tensor] = None,
                inputs_embeds: Optional[torch.Tensor] = None, past_key_values=None,
                labels: Optional[torch.LongTensor] = None, use_cache: Optional[bool] = None,
                output_attentions: Optional[bool] = None, output_hidden_states: Optional[bool] = None,
                return_dict: Optional[bool] = None, last_token_only: bool = False
                ) -> Union[Tuple, CausalLMOutputWithPast]:
        """As the reference's forward (:356-409).  `last_token_only=True` (an addition) computes logits for
        the final position only, which is all a generation loop needs after a long prefill."""
        if labels is not None:
            raise NotImplementedError("the training loss is outside the inference hot path")
        if return_dict is None:
            return_dict = bool(getattr(self.config, "return_dict", True))
        if use_cache is None:
            use_cache = self.config.use_cache if not self.training else False
        if self._can_fuse(input_ids, inputs_embeds, attention_mask, output_hidden_states):
            logits, cache = self._forward_fused(input_ids, inputs_embeds, past_key_values, use_cache, last_token_only,
                                                attention_mask)
            if not return_dict:
                return tuple(x for x in (logits, cache) if x is not None)
            return CausalLMOutputWithPast(loss=None, logits=logits, past_key_values=cache, hidden_states=None,
                                          attentions=None)
        outputs = self.model(input_ids=input_ids, attention_mask=attention_mask, inputs_embeds=inputs_embeds,
                             past_key_values=past_key_values, use_cache=use_cache,
                             output_attentions=output_attentions, output_hidden_states=output_hidden_states,
                             return_dict=True)
        hidden_states = outputs.last_hidden_state
        if last_token_only:
            hidden_states = hidden_states[:, -1:]
        logits = self.lm_head(hidden_states)
        if not return_dict:
            return tuple(x for x in (logits, outputs.past_key_values, outputs.hidden_states) if x is not None)
        return CausalLMOutputWithPast(loss=None, logits=logits, past_key_values=outputs.past_key_values,
                                      hidden_states=outputs.hidden_states, attentions=None)

    GREEDY_DECODERS = 2    # decoders (static state + captured step graph) kept per model, one per batch size

    @torch.no_grad()
    def _generate_graph(self, input_ids, max_new_tokens, eos_token_id, attention_mask, pick=None):
        """Generation with every decode step replayed from a CUDA graph (an eager step is about 200 launches
        through Python, several times what the GPU needs).  Same tokens as the step-by-step loop of `generate`:
        sequences are independent, so a finished sequence may keep running; its tokens after the first
        `eos_token_id` are overwritten with it, and the result is cut where the loop would have stopped.
        `pick` (sampling) maps the step's logits [B, V] to tokens [B]; None takes the graph's own arg-max.  Sampling
        draws its random numbers in the same order as the step loop, so both give the same tokens."""
        from ...engine import GreedyDecoder, fused_runner
        B = input_ids.shape[0]
        key = fused_runner(self).key
        decs = self.__dict__.get("_greedy_decoders")
        if decs is None or decs.get("key") != key:        # weights replaced or repacked: captured graphs are stale
            decs = {"key": key}
            object.__setattr__(self, "_greedy_decoders", decs)
        dec = decs.pop(B, None)
        if dec is None:
            dec = GreedyDecoder(self, B)
            while len(decs) - 1 >= self.GREEDY_DECODERS:
                decs.pop(next(k for k in decs if k != "key"))
        decs[B] = dec                                       # most recently used last
        if attention_mask is None and pick is None:
            dec.prefill(input_ids)
        else:
            out = self(input_ids=input_ids, attention_mask=attention_mask, use_cache=True, last_token_only=True)
            dec.seed(out.past_key_values, out.logits[:, -1])
            if pick is not None:
                dec.next.copy_(pick(out.logits[:, -1]))
        toks = torch.empty(B, max_new_tokens, dtype=torch.int64, device=input_ids.device)
        n = 0
        while n < max_new_tokens:
            toks[:, n].copy_(dec.next)
            n += 1
            if n == max_new_tokens:
                break
            if eos_token_id is not None and n % 16 == 0 and bool((toks[:, :n] == eos_token_id).any(dim=1).all()):
                break                                       # every sequence has finished (checked every 16 steps)
            dec.step()
            if pick is not None:
                dec.next.copy_(pick(dec.last_logits))
        toks = toks[:, :n]
        if eos_token_id is not None:
            hit = toks == eos_token_id
            after = (hit.cumsum(dim=1) - hit.to(torch.int64)) > 0          # positions after a sequence's first eos
            toks = torch.where(after, torch.full_like(toks, eos_token_id), toks)
            if bool(hit.any(dim=1).all()):                  # the step loop stops once the last sequence emits eos
                first = torch.where(hit, torch.arange(n, device=toks.device).expand_as(hit), n).min(dim=1).values
                toks = toks[:, : int(first.max().item()) + 1]
        return torch.cat([input_ids, toks], dim=1)

    # -- fused execution -------------------------------------------------------------------------------------
    fuse = True   # set False to run module by module (same kernels, unfused; used to cross-check the fused chain)

    def _can_fuse(self, input_ids, inputs_embeds, attention_mask, output_hidden_states) -> bool:
        if not self.fuse or (input_ids is None) == (inputs_embeds is None):
            return False
        if output_hidden_states or (output_hidden_states is None and getattr(self.config, "output_hidden_states", False)):
            return False
        if self.config.expand_ratio != 1 or self.config.hidden_size % 16 or self.config.intermediate_size is not None \
                and self.config.intermediate_size % 16:
            return False
        return True

    def _forward_fused(self, input_ids, inputs_embeds, past_key_values, use_cache, last_token_only, attention_mask=None):
        from ...engine import fused_runner
        ref = input_ids if input_ids is not None else inputs_embeds
        B = ref.shape[0]
        layers = self.model.layers
        if use_cache and past_key_values is not None:
            cache = past_key_values if isinstance(past_key_values, RecurrentCache) \
                else RecurrentCache.from_legacy_cache(past_key_values)
        else:
            cache = RecurrentCache.from_legacy_cache([layer.attn.init_state(B) for layer in layers])
        # The kernels advance float32 states in place.  A cache built the reference's way holds its states in the
        # parameter dtype (init_state: param.new_zeros; fused_recurrent_hgrn returns x.dtype): such states are widened
        # for the pass and written back, rounded to their own dtype, afterwards — the reference's rounding point.
        given = [cache.states[i][-1] for i in range(len(layers))]
        states = [s if s.dtype == torch.float32 else s.float() for s in given]
        logits, _ = fused_runner(self).forward(input_ids, inputs_embeds, states, last_token_only,
                                               attention_mask=attention_mask)
        for dst, src in zip(given, states):
            if dst is not src:
                dst.copy_(src)
        if use_cache and past_key_values is not None and len(layers):
            cache._seen_tokens += ref.shape[1]
        return logits, (cache.to_legacy_cache() if use_cache else None)

    @torch.no_grad()
    def generate(self, input_ids: torch.LongTensor, max_new_tokens: int = 20, max_length: Optional[int] = None,
                 do_sample: bool = False, eos_token_id: Optional[int] = None, top_p: float = 1.0, temperature: float = 1.0,
                 generator: Optional[torch.Generator] = None, attention_mask: Optional[torch.Tensor] = None,
                 use_graph: bool = True, **kwargs) -> torch.LongTensor:
        """Prefill once, then one cached single-token forward per new token; greedy, or with `do_sample=True` nucleus
        sampling (temperature, then top-p, as `generate.py:11` of the reference asks of transformers).

        The reference defers to transformers' GenerationMixin (:311-324), which current transformers releases
        no longer provide to this class.  Sampling draws one uniform number per sequence and step from `generator`
        (a CUDA generator; the default one if None) and is deterministic given those.  `attention_mask` marks
        left padding of the prompt.  Greedy decoding replays each step from a CUDA graph (`use_graph=False` runs the
        same kernels step by step).  Returns [B, prompt + new] token ids like GenerationMixin.generate."""
        # The reference hands every other option to transformers' GenerationMixin (:311-324).  Options that would change
        # the result and are not implemented here are refused instead of being silently ignored; the neutral value of
        # an option (what GenerationMixin does when it is absent) is accepted.
        neutral = {"num_beams": (1,), "top_k": (None, 0), "repetition_penalty": (None, 1.0), "min_length": (None, 0),
                   "min_new_tokens": (None, 0), "num_return_sequences": (None, 1), "length_penalty": (None, 1.0),
                   "no_repeat_ngram_size": (None, 0), "use_cache": (None, True), "return_dict_in_generate": (None, False),
                   "output_scores": (None, False), "output_hidden_states": (None, False), "output_attentions": (None, False),
                   "stopping_criteria": (None,), "logits_processor": (None,), "num_beam_groups": (None, 1),
                   "penalty_alpha": (None,), "typical_p": (None, 1.0), "bad_words_ids": (None,), "pad_token_id": None}
        for name, value in kwargs.items():
            if name not in neutral:
                raise NotImplementedError(f"generate(): option `{name}` is not implemented (greedy decoding and temperature / "
                                          f"top-p sampling with eos_token_id, max_new_tokens / max_length are)")
            allowed = neutral[name]
            if allowed is not None and not any(value is a or value == a for a in allowed):
                raise NotImplementedError(f"generate(): `{name}={value!r}` is not implemented (only {allowed[-1]!r})")
        pad_token_id = kwargs.get("pad_token_id")
        if pad_token_id is not None and eos_token_id is not None and pad_token_id != eos_token_id:
            raise NotImplementedError("generate(): finished sequences are padded with eos_token_id; a different pad_token_id "
                                      "is not implemented")

        def pick(logits):
            if not do_sample:
                return kernels.argmax_rows(logits)
            u = torch.rand(logits.shape[0], device=logits.device, dtype=torch.float32, generator=generator)
            return kernels.sample_top_p(logits, temperature, top_p, u)

        if max_length is not None:
            max_new_tokens = max(0, max_length - input_ids.shape[1])
        if use_graph and max_new_tokens > 0 and input_ids.is_cuda and self._can_fuse(input_ids, None, attention_mask, None):
            return self._generate_graph(input_ids, max_new_tokens, eos_token_id, attention_mask, pick if do_sample else None)
        out = self(input_ids=input_ids, attention_mask=attention_mask, use_cache=True, last_token_only=True)
        cache = RecurrentCache.from_legacy_cache(out.past_key_values, input_ids.shape[1])
        tokens = [input_ids]
        finished = torch.zeros(input_ids.shape[0], dtype=torch.bool, device=input_ids.device)
        for step in range(max_new_tokens):
            nxt = pick(out.logits[:, -1])
            if eos_token_id is not None:
                nxt = torch.where(finished, torch.full_like(nxt, eos_token_id), nxt)
                finished |= nxt == eos_token_id
            tokens.append(nxt[:, None])
            if step + 1 == max_new_tokens or (eos_token_id is not None and bool(finished.all())):
                break
            out = self(input_ids=nxt[:, None], past_key_values=cache, use_cache=True)
        return torch.cat(tokens, dim=1)
