"""Generation: sampling, single-sequence serving (plain / Harmony chat REPL) and the batched
prefill + decode harness (lyra/generate.py:21-213).

Per-sequence semantics equal the reference's: greedy when temperature <= 0, otherwise logits / temperature,
exactly top-k candidates kept, categorical sample; prompts begin with eos; the per-token random stream is
derived from ``(seed, turn, token index)``. ``BatchedGenerator`` is the serving path for many sequences at once:
one prefill, then a decode loop whose per-token work is a fixed launch sequence (capturable in a CUDA graph),
with attention data-parallel over the batch and experts expert-parallel over the ranks.
"""

from __future__ import annotations

import codecs
import itertools
from dataclasses import dataclass, replace
from typing import Callable

import torch

from lyra_b200.config import Mode, ModelConfig
from lyra_b200.model import ModelCache, ModelWeights, model_apply
from lyra_b200.tokenizer import LyraTokenizer


@dataclass(frozen=True, kw_only=True)
class InferenceConfig:
    weights: str
    max_new_tokens: int = 256
    max_cache_length: int | None = None
    fp8: bool = False
    temperature: float | None = None
    top_k: int | None = None


def apply_inference_overrides(mcfg: ModelConfig, icfg: InferenceConfig) -> ModelConfig:
    """``--fp8`` quantises the MLP weights and the KV cache, not the attention projections (lyra/generate.py:31-38)."""
    if icfg.temperature is not None:
        mcfg = replace(mcfg, sample_temperature=icfg.temperature)
    if icfg.top_k is not None:
        mcfg = replace(mcfg, sample_topk=icfg.top_k)
    if icfg.fp8:
        mcfg = replace(mcfg, gemm_dtype=torch.float8_e4m3fn, quantize_mlp=True, quantize_cache=True)
    return mcfg


def load_model(mcfg: ModelConfig, icfg: InferenceConfig, device="cpu", rt=None) -> ModelWeights:
    mcfg = apply_inference_overrides(mcfg, icfg)
    return ModelWeights.quantize(ModelWeights.load(icfg.weights, mcfg, device=device, rt=rt), mcfg)


def _key(seed: int, *folds: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    s = seed & 0xFFFFFFFF
    for f in folds:
        s = (s * 0x9E3779B1 + (int(f) + 0x7F4A7C15)) & 0xFFFFFFFFFFFF
    g.manual_seed(s)
    return g


def sample_token(logits: torch.Tensor, key: torch.Generator | None, mcfg: ModelConfig) -> torch.Tensor:
    """One token id from ``logits [V]`` (or ``[B, V]`` -> ``[B]``)."""
    if mcfg.sample_temperature <= 0:
        return torch.argmax(logits, dim=-1).to(torch.int32)
    z = logits.float() / mcfg.sample_temperature
    if 0 < mcfg.sample_topk < z.shape[-1]:
        vals, idx = torch.sort(z, dim=-1, descending=True, stable=True)  # ties -> lower index, like lax.top_k
        vals, idx = vals[..., : mcfg.sample_topk], idx[..., : mcfg.sample_topk]
        probs = torch.softmax(vals, dim=-1)
        pick = torch.multinomial(probs.cpu().reshape(-1, probs.shape[-1]), 1, generator=key).reshape(probs.shape[:-1] + (1,))
        return idx.gather(-1, pick.to(idx.device)).squeeze(-1).to(torch.int32)
    probs = torch.softmax(z, dim=-1)
    pick = torch.multinomial(probs.cpu().reshape(-1, probs.shape[-1]), 1, generator=key).reshape(probs.shape[:-1])
    return pick.to(logits.device).to(torch.int32)


@torch.no_grad()
def generate(ctx: torch.Tensor, model: ModelWeights, cache: ModelCache, key, mcfg: ModelConfig, sample_pos: int, rt=None):
    """One model call + one sampled token for a single sequence ``ctx [1, T]`` (lyra/generate.py:56-61)."""
    logits, _, updated = model_apply(ctx, model, cache, mcfg, rt=rt)
    token = sample_token(logits[0, sample_pos], key, mcfg)
    if getattr(rt, "tp_size", 1) > 1:      # the ranks of a model axis must feed back the same token: rank 0's draw is the one that counts
        import torch.distributed as dist

        dist.broadcast(token, src=dist.get_global_rank(rt.group, 0) if rt.group is not None else 0, group=rt.group)
    return token, updated


def init_cache(mcfg: ModelConfig, length: int, device="cpu", batch: int = 1, n_kv_local: int | None = None) -> ModelCache:
    return ModelCache.create(mcfg, batch, length, device, n_kv_local)


@torch.no_grad()
def sample_tokens(model: ModelWeights, seed_key: tuple[int, ...], mcfg: ModelConfig, prompt: list[int], max_new_tokens: int,
                  device="cpu", rt=None) -> list[int]:
    """Prefill + token-by-token decode on the device; returns ``max_new_tokens`` ids (lyra/generate.py:64-85)."""
    prefill, decode = replace(mcfg, mode=Mode.PREFILL), replace(mcfg, mode=Mode.DECODE)
    n = len(prompt)
    cache = init_cache(mcfg, n + max_new_tokens, device, n_kv_local=getattr(rt, "n_kv_local", None))
    ctx = torch.tensor([prompt], dtype=torch.long, device=device)
    token, cache = generate(ctx, model, cache, _key(*seed_key, 0), prefill, n - 1, rt)
    cache.pos = n
    out = [int(token)]
    for index in range(1, max_new_tokens):
        token, cache = generate(token.reshape(1, 1).long(), model, cache, _key(*seed_key, index), decode, 0, rt)
        out.append(int(token))
    return out


def sample_eval_step(model: ModelWeights, prompt: list[int], sample_index: int, max_new_tokens: int, mcfg: ModelConfig, device="cpu", rt=None):
    """Training-time sampling with the run's fixed random stream (lyra/training/steps.py:94-99)."""
    return sample_tokens(model, (mcfg.seed, 1, sample_index), mcfg, prompt, max_new_tokens, device, rt)


# --------------------------------------------------------------------------- batched serving harness
class BatchedGenerator:
    """Batched prefill + greedy/sampled decode. ``prompts [B, P]`` are equal-length token rows on this rank; with an
    expert-parallel runtime every rank serves its own rows and the experts are shared across ranks.

    ``prefill`` returns the first generated token per row and its duration; ``decode`` runs ``n`` further tokens.
    With ``use_cuda_graph`` the per-token launch sequence is captured once and replayed."""

    def __init__(self, model: ModelWeights, mcfg: ModelConfig, *, batch: int, capacity: int, device, rt=None, use_cuda_graph: bool = False):
        self.model, self.rt, self.device = model, rt, torch.device(device)
        self.prefill_cfg = replace(mcfg, mode=Mode.PREFILL)
        self.decode_cfg = replace(mcfg, mode=Mode.DECODE)
        self.cache = init_cache(mcfg, capacity, device, batch, getattr(rt, "n_kv_local", None))   # tensor parallel: this rank's kv heads only
        self.batch, self.capacity = batch, capacity
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        # The expert exchange alternates between two count buffers from call to call; a graph fixes each call's buffer at capture.
        # With an odd number of exchanges per token the last call of one replay and the first call of the next would share a
        # buffer, which the protocol does not allow: such models decode without a graph under expert parallelism.
        if rt is not None and getattr(rt, "ep_size", 1) > 1 and sum(kind == "moe" for kind in mcfg.mlp_map) % 2 == 1:
            self.use_cuda_graph = False
        self._graph = None
        self._static_tok = None
        self._static_out = None

    @torch.no_grad()
    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        B, P = prompts.shape
        self.cache.pos = 0
        hidden, _, self.cache = model_apply(prompts.long(), self.model, self.cache, self.prefill_cfg, return_hidden_states=True, rt=self.rt)
        return self._next_from_hidden(hidden[:, -1])

    def _next_from_hidden(self, h_last: torch.Tensor) -> torch.Tensor:
        from lyra_b200.model import lm_head_weight

        cfg = self.decode_cfg
        unemb = lm_head_weight(self.model.tok, cfg)
        if self.rt is not None:
            unemb = self.rt.materialize(unemb)
        logits = (h_last @ unemb.to(h_last.dtype).t()).float()
        logits[..., cfg.vocab_size:] = float("-inf")
        return sample_token(logits, None if cfg.sample_temperature <= 0 else _key(cfg.seed, self.cache.pos), cfg)

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        hidden, _, self.cache = model_apply(tokens.reshape(self.batch, 1).long(), self.model, self.cache, self.decode_cfg,
                                            return_hidden_states=True, rt=self.rt)
        return self._next_from_hidden(hidden[:, -1])

    @torch.no_grad()
    def decode(self, first: torch.Tensor, n: int) -> torch.Tensor:
        if self.use_cuda_graph and self.decode_cfg.sample_temperature <= 0 and (self.rt is None or getattr(self.rt, "implementation", "") == "b200"):
            return self._decode_graph(first, n)
        out = [first]
        tok = first
        for _ in range(n - 1):
            tok = self.decode_step(tok)
            out.append(tok)
        return torch.stack(out, dim=1)

    def _graph_step(self) -> None:
        """One greedy token from ``_static_tok`` at the device-resident position; advances both in place."""
        hidden, _, cache = model_apply(self._static_tok.reshape(self.batch, 1), self.model, self.cache, self.decode_cfg,
                                       return_hidden_states=True, rt=self.rt)
        nxt = self._next_from_hidden(hidden[:, -1])
        self._static_tok.copy_(nxt)
        self.cache.pos_dev.add_(1)

    @torch.no_grad()
    def _decode_graph(self, first: torch.Tensor, n: int) -> torch.Tensor:
        """Greedy decode with the per-token launch sequence captured once in a CUDA graph and replayed: the position
        lives in device memory (cache writes, RoPE row, attention bounds read it there), so every replay is identical
        on the host side and costs one launch instead of a few hundred. With an expert-parallel runtime the exchange kernels
        are part of the graph (their epochs are device counters), and every rank replays the same number of times."""
        start = self.cache.pos
        if start + n - 1 > self.capacity:
            raise ValueError(f"cache capacity {self.capacity} too small for {start} + {n - 1} positions")
        if self._graph is None:
            self._static_tok = torch.zeros(self.batch, dtype=torch.long, device=self.device)
            self.cache.pos_dev = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._out = None
            # a first eager step on a side stream: one-time kernel set-up and allocator warm-up must not be captured
            self._static_tok.copy_(first)
            self.cache.pos_dev.fill_(start)
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self._graph_step()
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            self._graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self._graph):
                self._graph_step()
        self._static_tok.copy_(first)
        self.cache.pos_dev.fill_(start)
        out = torch.empty(self.batch, n, dtype=torch.long, device=self.device)
        out[:, 0] = first
        for i in range(1, n):
            self._graph.replay()
            out[:, i] = self._static_tok
        self.cache.pos = start + n - 1
        return out


# --------------------------------------------------------------------------- REPL
def serve_model(model: ModelWeights, mcfg: ModelConfig, icfg: InferenceConfig, *, harmony: bool = False, device="cpu", rt=None,
                input_fn: Callable[[str], str] = input, output_fn: Callable[..., None] = print) -> None:
    """Interactive chat loop, one sequence, one device call per token (lyra/generate.py:130-213)."""
    mcfg = apply_inference_overrides(mcfg, icfg)
    capacity = icfg.max_cache_length or mcfg.seq_len
    prefill_cfg, decode_cfg = replace(mcfg, mode=Mode.PREFILL), replace(mcfg, mode=Mode.DECODE)
    tokenizer = LyraTokenizer()

    if harmony:
        from openai_harmony import Conversation, HarmonyEncodingName, Message, Role, StreamableParser, load_harmony_encoding

        encoding = load_harmony_encoding(HarmonyEncodingName.HARMONY_GPT_OSS)
        stop_tokens = set(encoding.stop_tokens_for_assistant_actions())
        user_turn = lambda prompt: [Message.from_role_and_content(Role.USER, prompt)]
        reply_turns = lambda tokens: encoding.parse_messages_from_completion_tokens(tokens, Role.ASSISTANT, strict=False)
        render = lambda turns: encoding.render_conversation_for_completion(Conversation.from_messages(turns), Role.ASSISTANT)

        def text_stream():
            parser = StreamableParser(encoding, Role.ASSISTANT, strict=False)

            def final_channel(token):
                if token is None:
                    return ""
                parser.process(token)
                return (parser.last_content_delta or "") if parser.current_channel == "final" else ""

            return final_channel
    else:
        stop_tokens = {tokenizer.eos_token}
        user_turn = lambda prompt: [[tokenizer.eos_token, *tokenizer.encode_ordinary(prompt)]]
        reply_turns = lambda tokens: [tokens]
        render = lambda turns: [t for turn in turns for t in turn]

        def text_stream():
            decoder = codecs.getincrementaldecoder("utf-8")(errors="replace")
            return lambda token: decoder.decode(b"" if token is None else tokenizer.decode_single_token_bytes(token), final=token is None)

    output_fn("Type a prompt to talk to the model. Ctrl-D or 'exit' to quit.\n")
    turns: list = []
    for turn in itertools.count():
        try:
            prompt = input_fn("User: ").strip()
        except EOFError:
            break
        if prompt in ("exit", "quit"):
            break
        if not prompt:
            continue
        context = render([*turns, *user_turn(prompt)])
        if len(context) >= capacity:
            turns, context = [], render(user_turn(prompt))
            if len(context) >= capacity:
                output_fn(f"\n[the prompt needs {len(context)} tokens but the context window is {capacity}]\n")
                continue
            output_fn("\n[context window full; starting a new conversation]\n")

        cache = init_cache(mcfg, capacity, device, n_kv_local=getattr(rt, "n_kv_local", None))
        ctx = torch.tensor([context], dtype=torch.long, device=device)
        token, cache = generate(ctx, model, cache, _key(mcfg.seed, turn, -1), prefill_cfg, len(context) - 1, rt)
        cache.pos = len(context)
        output_fn()
        to_text, reply = text_stream(), []
        for index in range(min(icfg.max_new_tokens, capacity - len(context))):
            next_token = int(token)
            if next_token in stop_tokens:
                break
            reply.append(next_token)
            output_fn(to_text(next_token), end="", flush=True)
            token, cache = generate(torch.tensor([[next_token]], dtype=torch.long, device=device), model, cache,
                                    _key(mcfg.seed, turn, index), decode_cfg, 0, rt)
        output_fn(to_text(None) + "\n")
        turns = [*turns, *user_turn(prompt), *reply_turns(reply)]
