"""Model backends of the OpenAI server: the native Qwen engine and the GGUF runtimes, each
paired with a chat tokenizer."""
from __future__ import annotations

from pathlib import Path
from typing import Iterator, Sequence

import torch

from ..encoding import chat, dsv4, gguf_tokenizer
from .engine import SamplingParams, apply_penalties, sample_token, token_logprobs


class QwenBackend:
    """Greedy requests run on the engine's CUDA-graph decode in bursts; sampled requests read
    the logits back after every step."""

    def __init__(self, engine, burst: int = 8, speculator=None):
        """`speculator`: a `QwenDSparkSpeculator` over the same engine; greedy requests then run as block-drafted speculative
        rounds (same tokens as plain greedy decode)."""
        self.eng, self.burst, self.spec = engine, burst, speculator

    def generate(self, prompt_ids: Sequence[int], p: SamplingParams) -> Iterator[int]:
        eng = self.eng
        eng.reset()
        plain = p.temperature <= 0 and p.repetition_penalty == 1.0 and p.frequency_penalty == 0 and p.presence_penalty == 0
        if self.spec is not None and plain and p.logprobs < 0:
            first = self.spec.prefill(list(prompt_ids))
            yield first
            n, last = 1, first
            while n < p.max_tokens and last not in p.stop_token_ids:
                for t in self.spec.decode(last, min(self.burst, p.max_tokens - n)):
                    n += 1
                    last = t
                    yield t
                    if t in p.stop_token_ids:
                        return
            return
        if p.logprobs >= 0:
            # every step's logits come back to the host: sample there and report the model's log-probabilities
            if getattr(eng, "tp_world", 1) > 1:
                raise RuntimeError("log-probabilities need the whole vocabulary on one rank (logits are vocabulary shards under tensor parallelism)")
            gen = torch.Generator().manual_seed(p.seed) if p.seed is not None else None
            eng.prefill(list(prompt_ids))
            produced: list[int] = []
            while True:
                raw = eng.logits(0)
                t = sample_token(apply_penalties(raw.clone(), produced, p), p, gen)
                produced.append(t)
                yield token_logprobs(raw, t, p.logprobs)
                if len(produced) >= p.max_tokens or t in p.stop_token_ids:
                    return
                eng.forward_rows([t])
        tok = eng.prefill(list(prompt_ids))
        produced = [tok]
        yield tok
        greedy = p.temperature <= 0 and p.repetition_penalty == 1.0 and p.frequency_penalty == 0 and p.presence_penalty == 0
        gen = torch.Generator().manual_seed(p.seed) if p.seed is not None else None
        while len(produced) < p.max_tokens and produced[-1] not in p.stop_token_ids:
            if greedy:
                n = min(self.burst, p.max_tokens - len(produced))
                for t in eng.decode(n, sync_each_step=False):
                    produced.append(t)
                    yield t
                    if t in p.stop_token_ids:
                        return
            else:
                # re-run the last position's logits through the host sampler
                logits = apply_penalties(eng.logits(0), produced, p)
                t = sample_token(logits, p, gen)
                produced[-1] = t
                eng_next = eng.forward_rows([t])[0]
                produced.append(eng_next)
                yield eng_next


class GGUFBackend:
    def __init__(self, runtime):
        self.rt = runtime

    def generate(self, prompt_ids: Sequence[int], p: SamplingParams) -> Iterator[int]:
        self.rt.reset()
        greedy = p.temperature <= 0 and p.repetition_penalty == 1.0 and p.frequency_penalty == 0 and p.presence_penalty == 0
        if p.logprobs >= 0 or not greedy:
            # sampled or penalised requests, and log-probability reports, take every step's logits through the host sampler
            if not hasattr(self.rt, "forward_logits"):
                raise RuntimeError("this runtime does not expose logits: sampling and log-probabilities are not available")
            gen = torch.Generator().manual_seed(p.seed) if p.seed is not None else None
            raw = self.rt.forward_logits(list(prompt_ids))
            produced: list[int] = []
            while True:
                t = sample_token(apply_penalties(raw.clone(), produced, p), p, gen)
                produced.append(t)
                yield token_logprobs(raw, t, p.logprobs) if p.logprobs >= 0 else t
                if len(produced) >= p.max_tokens or t in p.stop_token_ids:
                    return
                raw = self.rt.forward_logits([t])
        tok = self.rt.prefill(list(prompt_ids))
        n = 1
        yield tok
        while n < p.max_tokens and tok not in p.stop_token_ids:
            tok = self.rt.decode_one(tok)
            n += 1
            yield tok


class DSV4Backend:
    """DeepSeek-V4 runtime (`models.deepseek_v4_runtime.DSV4Runtime`): prefill, then one row per step; sampled requests
    take the logits of each step through the host sampler."""

    def __init__(self, runtime):
        self.rt = runtime

    def generate(self, prompt_ids: Sequence[int], p: SamplingParams) -> Iterator[int]:
        rt = self.rt
        rt.reset()
        greedy = p.temperature <= 0 and p.repetition_penalty == 1.0 and p.frequency_penalty == 0 and p.presence_penalty == 0
        gen = torch.Generator().manual_seed(p.seed) if p.seed is not None else None
        logits = rt.forward_logits(list(prompt_ids))[-1]
        produced: list[int] = []
        while True:
            tok = int(torch.argmax(logits)) if greedy else sample_token(apply_penalties(logits.clone(), produced, p), p, gen)
            rt.combine.check_step("cuda")
            produced.append(tok)
            yield token_logprobs(logits, tok, p.logprobs) if p.logprobs >= 0 else tok
            if len(produced) >= p.max_tokens or tok in p.stop_token_ids:
                return
            logits = rt.forward_logits([tok])[-1]


class HFChatTokenizer:
    """`tokenizers.Tokenizer` + a chat renderer + a completion parser."""

    def __init__(self, tok, render, eos_ids: Sequence[int], parse=None):
        self.tok, self.render, self._eos, self._parse = tok, render, tuple(eos_ids), parse

    def encode_chat(self, messages, *, tools=None, thinking=False, reasoning_effort=None, response_format=None):
        text = self.render(messages, tools=tools, thinking=thinking, reasoning_effort=reasoning_effort, response_format=response_format)
        return self.tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids):
        return self.tok.decode(list(ids), skip_special_tokens=False)

    def parse(self, text: str, thinking: bool) -> dict:
        if self._parse:
            return self._parse(text, thinking)
        r, v = chat.split_thinking(text)
        msg = {"role": "assistant", "content": v}
        if r:
            msg["reasoning_content"] = r
        return msg

    @property
    def eos_ids(self):
        return self._eos


def build(kind: str, ckpt: str, max_context: int, qwen_dspark: str | None = None, tokenizer_path: str | None = None,
          layer_pipeline: bool = False, speculative: tuple[str, int] = ("off", 4)):
    """(backend, tokenizer) for `--model qwen|gguf|dsv4`. Under torchrun every rank builds its shard (rank and world come
    from the environment). `tokenizer_path`: directory with tokenizer.json when it is not the checkpoint directory.
    `layer_pipeline` (dsv4, several ranks): contiguous layer ranges per rank instead of expert parallelism.
    `speculative` = (mode, draft length) of the typed configuration: `ngram` gives the Qwen backend a prompt-lookup drafter
    (greedy requests run as draft + verify rounds with the same tokens as plain decoding)."""
    import os
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    if kind == "dsv4":
        from tokenizers import Tokenizer
        from ..models import deepseek_v4_loader as loader
        from ..models.deepseek_v4_runtime import DSV4Runtime
        raw_experts = None
        if str(ckpt).endswith(".gguf"):
            # deepseek4 GGUF: dense tensors dequantised on load, routed experts kept as raw blocks; the tokenizer needs a directory
            from ..models import deepseek_v4_gguf as dg
            cfg, weights, raw_experts = dg.load_gguf(ckpt)
            if not tokenizer_path:
                raise ValueError("a deepseek4 GGUF checkpoint needs --tokenizer-path (a directory with tokenizer.json)")
        else:
            cfg, weights = loader.load_checkpoint(ckpt)
        if layer_pipeline and world > 1:
            from ..parallel.pipeline import PipelineStage
            rt = DSV4Runtime(cfg, weights, max_context=max_context, pipeline=PipelineStage(cfg.n_layers), raw_experts=raw_experts)
        else:
            rt = DSV4Runtime(cfg, weights, max_context=max_context, rank=rank, world=world, raw_experts=raw_experts)
        tok = Tokenizer.from_file(str(Path(tokenizer_path or ckpt) / "tokenizer.json"))
        eos = [i for i in (tok.token_to_id(dsv4.EOS),) if i is not None]

        def render(messages, *, tools=None, thinking=False, reasoning_effort=None, response_format=None, **_):
            return dsv4.encode_messages(messages, tools=tools, thinking_mode="thinking" if thinking else "chat",
                                        reasoning_effort=reasoning_effort, response_format=response_format)
        parse = lambda text, thinking: dsv4.parse_completion(("<think>" if thinking else "") + text, "thinking" if thinking else "chat")
        return DSV4Backend(rt), HFChatTokenizer(tok, render, eos, parse)
    if kind == "qwen":
        from tokenizers import Tokenizer
        from ..models import qwen_hybrid as qh
        cfg = qh.QwenHybridConfig.from_json((Path(ckpt) / "config.json").read_text())
        eng = qh.QwenEngine(cfg, tp_rank=rank, tp_world=world, device=local, max_context=max_context).load(ckpt)
        if world > 1:
            from ..parallel import tp
            tp.connect_engine(eng)
        tok = Tokenizer.from_file(str(Path(tokenizer_path or ckpt) / "tokenizer.json"))
        eos = [i for i in (tok.token_to_id("<|im_end|>"), tok.token_to_id("<|endoftext|>")) if i is not None]

        def render(messages, *, tools=None, thinking=False, **_):
            out = ""
            for m in messages:
                out += f"<|im_start|>{m['role']}\n{dsv4._text(m.get('content'))}<|im_end|>\n"
            return out + "<|im_start|>assistant\n" + ("<think>\n" if thinking else "")
        spec = None
        if qwen_dspark:
            # external block drafter (one rank): its layers run on the GPU next to the engine, coupled through target taps
            if world > 1:
                raise ValueError("--qwen-dspark runs on one rank (the target taps are captured on one rank)")
            from ..formats import safetensors_io as st_io
            from ..models import qwen_dspark as qd
            from ..models.qwen_dspark_runtime import QwenDSparkRuntime, QwenDSparkSpeculator
            dcfg, dw = qd.load_checkpoint(qwen_dspark)
            dcfg.validate_for_target(cfg.hidden_size, cfg.vocab_size, cfg.num_hidden_layers)
            model = st_io.SafetensorsModel(ckpt)
            names = set(model.keys())
            embed_name = next(n for n in ("model.language_model.embed_tokens.weight", "model.embed_tokens.weight") if n in names)
            embed = model.get(embed_name)
            lm_head = model.get("lm_head.weight") if "lm_head.weight" in names else embed
            spec = QwenDSparkSpeculator(eng, QwenDSparkRuntime(dcfg, dw, embed, lm_head, max_context=max_context, device=f"cuda:{local}"))
        if spec is None and speculative[0] == "ngram":
            from ..runtime.speculative import DrafterSpeculator, NGramDrafter
            spec = DrafterSpeculator(eng, NGramDrafter(), k=max(1, min(int(speculative[1]), 7)))
        return QwenBackend(eng, speculator=spec), HFChatTokenizer(tok, render, eos)
    from ..models import registry
    md = gguf_tokenizer.read_metadata(ckpt)
    tok = gguf_tokenizer.build_tokenizer(md)
    arch = md.get("general.architecture")
    rt = registry.build_runtime(ckpt, max_context=max_context)
    sp = gguf_tokenizer.special_ids(md)
    eos = [i for i in (sp["eos"], sp["eot"]) if i is not None]
    if arch == "glm-dsa":
        render = lambda messages, *, thinking=False, **_: chat.render_glm(messages, thinking=thinking)
    else:
        render = lambda messages, *, thinking=False, **_: chat.render_minimax(messages, thinking=thinking)
    return GGUFBackend(rt), HFChatTokenizer(tok, render, eos)


def build_tokenizer(kind: str, path: str, chat_format: str = "qwen"):
    """Chat tokenizer alone (no model): `hf` = a directory with tokenizer.json, `gguf` = a GGUF file's metadata.
    chat_format: qwen | glm | minimax | dsv4."""
    if kind == "hf":
        from tokenizers import Tokenizer
        tok = Tokenizer.from_file(str(Path(path) / "tokenizer.json"))
        names = {"qwen": ("<|im_end|>", "<|endoftext|>"), "dsv4": (dsv4.EOS,)}.get(chat_format, ("</s>",))
        eos = [i for i in (tok.token_to_id(n) for n in names) if i is not None]
    else:
        md = gguf_tokenizer.read_metadata(path)
        tok = gguf_tokenizer.build_tokenizer(md)
        sp = gguf_tokenizer.special_ids(md)
        eos = [i for i in (sp["eos"], sp["eot"]) if i is not None]

    def render(messages, *, tools=None, thinking=False, reasoning_effort=None, response_format=None, **_):
        if chat_format == "glm":
            return chat.render_glm(messages, thinking=thinking)
        if chat_format == "minimax":
            return chat.render_minimax(messages, thinking=thinking)
        if chat_format == "dsv4":
            return dsv4.encode_messages(messages, tools=tools, thinking_mode="thinking" if thinking else "chat",
                                        reasoning_effort=reasoning_effort, response_format=response_format)
        out = ""
        for m in messages:
            out += f"<|im_start|>{m['role']}\n{dsv4._text(m.get('content'))}<|im_end|>\n"
        return out + "<|im_start|>assistant\n" + ("<think>\n" if thinking else "")
    parse = (lambda text, thinking: dsv4.parse_completion(("<think>" if thinking else "") + text, "thinking" if thinking else "chat")) \
        if chat_format == "dsv4" else None
    return HFChatTokenizer(tok, render, eos, parse)
