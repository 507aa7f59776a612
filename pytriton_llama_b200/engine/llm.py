"""Python entry points: token ids in, token ids out, through scheduler, step function and sampler.

``LLM`` is the engine-level interface.  ``GenerateText`` and ``GenerateStreamText`` keep the names
and the meaning of the arguments of lite_llama's classes (lite_llama/generate.py:52-61,87-95,
156-177; lite_llama/generate_stream.py:55-64,90-98,190-216): ``checkpoints_dir``,
``tokenizer_path``, ``max_seq_len``, ``max_gpu_num_blocks``, ``compiled_model``, ``device``;
``generate(prompt_tokens, max_gen_len, temperature, top_p, echo)``.  ``load_model`` and
``triton_weight`` are accepted and ignored: weights are always read from the folder's
safetensors files and there are no Triton kernels.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Generator, Hashable, Iterable, List, Optional, Sequence, Tuple, Union

import torch

from ..config.engine import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .engine import Engine, StepEntry
from .scheduler import PENDING, Request, Scheduler, StepPlan


@dataclass
class _Launched:
    """A step that runs on the device, and where its tokens will arrive on the host."""
    plan: StepPlan
    requests: List[Request]              # one per sampled row, in row order
    host: Optional[torch.Tensor] = None  # int32 [2, rows]: tokens, bit patterns of the log-probabilities
    event: object = None
    logprobs: bool = False


class LLM:
    def __init__(self, model_dir, config: Optional[EngineConfig] = None, device="cuda:0", ops=None, **engine_options):
        """``engine_options`` go to ``Engine`` (``model_config`` and ``random_seed`` for random weights)."""
        self.engine = Engine(model_dir, config, device=device, ops=ops, **engine_options)
        cfg = self.engine.config
        self.scheduler = Scheduler(self.engine.cache, cfg.max_num_seqs, cfg.max_batched_tokens,
                                   cfg.max_seq_len, eos_token_ids=self.engine.eos_token_ids)
        self.sampler = Sampler(self.engine.ops, self.engine.device, seed=cfg.seed)
        self._next_id = 0
        self._rows: Dict[Hashable, int] = {}     # request -> its row among the tokens sampled by the last launched step
        self._turn = 0
        self._staging = []
        if self.engine.device.type == "cuda":
            # where sampled tokens arrive on the host; a buffer is read before the launch after next reuses it
            self._staging = [(torch.empty((2, cfg.max_num_seqs), dtype=torch.int32, pin_memory=True), torch.cuda.Event())
                             for _ in range(3)]

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    request_id: Optional[Hashable] = None) -> Request:
        if request_id is None:
            request_id = f"req-{self._next_id}"
            self._next_id += 1
        prompt = [int(t) for t in prompt]
        vocab = self.engine.vocab_size
        if any(t < 0 or t >= vocab for t in prompt):
            raise ValueError(f"the prompt has a token outside the vocabulary of {vocab}")
        return self.scheduler.add(request_id, prompt, params)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def step(self) -> Tuple[Dict[Hashable, int], List[Request]]:
        """Runs one scheduled step and reads its tokens.  Returns (request id -> new token, requests
        that finished)."""
        launched = self._launch()
        if launched is None:
            if self.scheduler.has_work():
                raise RuntimeError("the scheduler found nothing to run although requests are pending")
            return {}, []
        return self._collect(launched)

    def run(self) -> Generator[Tuple[Dict[Hashable, int], List[Request]], None, None]:
        """Steps until no request is left, yielding what ``step`` returns for every step.  With
        ``overlap_steps`` the next step is planned and launched before the tokens of the last one are
        read: a request that goes on takes its token on the device (``StepEntry.from_row``), so the
        host's work runs beside the device's.  The tokens are the same either way; a request that a
        stop token ends has by then run one step more, whose token is dropped."""
        overlap = self.engine.config.overlap_steps
        waiting_for: Optional[_Launched] = None
        while waiting_for is not None or self.scheduler.has_work():
            launched = self._launch()
            if launched is None and waiting_for is None:
                raise RuntimeError("the scheduler found nothing to run although requests are pending")
            if waiting_for is not None:
                yield self._collect(waiting_for)
                waiting_for = None
            if launched is not None and not overlap:
                yield self._collect(launched)
            else:
                waiting_for = launched

    def _launch(self) -> Optional[_Launched]:
        plan = self.scheduler.schedule()
        if not plan.portions:
            return _Launched(plan, []) if plan.finished else None
        entries = []
        for p in plan.portions:
            req = p.request
            if req.output and req.output[-1] == PENDING and p.start + p.length == len(req.prompt) + len(req.output):
                if p.length != 1:
                    raise RuntimeError(f"request {req.id!r}: a token that has not been read yet lies inside a longer portion")
                entries.append(StepEntry(req.id, [0], [0], from_row=self._rows[req.id]))
            else:
                entries.append(StepEntry(req.id, req.tokens(p.start, p.length), [p.length - 1] if p.sample else []))
        # the plan was checked against the cache and the tokens at intake; the logits are sampled from at once
        out = self.engine.step(entries, validate=False, own_logits=False)
        reqs = [p.request for p in plan.portions if p.sample]
        launched = _Launched(plan, reqs)
        if reqs:
            n = len(reqs)
            tokens, lp = self.sampler.sample_device(out.logits, [r.params for r in reqs], [r.number for r in reqs],
                                                    [len(r.output) for r in reqs], out=self.engine.sampled[:n])
            launched.logprobs = lp is not None
            if self.engine.device.type == "cuda":
                launched.host, launched.event = self._staging[self._turn % len(self._staging)]
                self._turn += 1
                launched.host[0, :n].copy_(tokens, non_blocking=True)
                if lp is not None:
                    launched.host[1, :n].view(torch.float32).copy_(lp, non_blocking=True)
                launched.event.record(torch.cuda.current_stream(self.engine.device))
            else:
                launched.host = torch.stack([tokens.cpu(), (lp if lp is not None else torch.zeros(n)).cpu().view(torch.int32)])
        self._rows = {r.id: i for i, r in enumerate(reqs)}
        self.scheduler.advance(plan)
        return launched

    def _collect(self, launched: _Launched) -> Tuple[Dict[Hashable, int], List[Request]]:
        finished = list(launched.plan.finished)
        reqs = launched.requests
        if not reqs:
            return {}, finished + self.scheduler.resolve(launched.plan, {})[1]
        if launched.event is not None:
            launched.event.synchronize()
        n = len(reqs)
        tokens = launched.host[0, :n].tolist()
        sampled = {r.id: t for r, t in zip(reqs, tokens)}
        logprobs = None
        if launched.logprobs:
            values = launched.host[1, :n].view(torch.float32).tolist()
            logprobs = {r.id: (v if r.params.logprobs else None) for r, v in zip(reqs, values)}
        accepted, done = self.scheduler.resolve(launched.plan, sampled, logprobs)
        return accepted, finished + done

    # ------------------------------------------------------------------ whole runs
    def generate(self, prompt_tokens: Sequence[Sequence[int]],
                 params: Union[None, SamplingParams, Sequence[SamplingParams]] = None) -> List[List[int]]:
        """Generated token ids of every prompt (without the prompt), in the order given."""
        plist = self._params_list(params, len(prompt_tokens))
        reqs = [self.add_request(p, sp) for p, sp in zip(prompt_tokens, plist)]
        for _ in self.run():
            pass
        self.engine.check_device_status()
        return [list(r.output) for r in reqs]

    def generate_stream(self, prompt_tokens: Sequence[Sequence[int]],
                        params: Union[None, SamplingParams, Sequence[SamplingParams]] = None
                        ) -> Generator[List[Tuple[int, List[int], bool]], None, None]:
        """Yields, after every step that produced tokens, a list of (prompt index, new token ids,
        finished)."""
        plist = self._params_list(params, len(prompt_tokens))
        reqs = [self.add_request(p, sp) for p, sp in zip(prompt_tokens, plist)]
        index = {r.id: i for i, r in enumerate(reqs)}
        early = [(index[r.id], [], True) for r in reqs if r.status == "finished"]
        if early:
            yield early
        for sampled, finished in self.run():
            done = {r.id for r in finished}
            events = [(index[rid], [tok], rid in done) for rid, tok in sampled.items() if rid in index]
            events += [(index[r.id], [], True) for r in finished if r.id in index and r.id not in sampled]
            if events:
                yield sorted(events)

    @staticmethod
    def _params_list(params, n: int) -> List[SamplingParams]:
        if params is None:
            return [SamplingParams() for _ in range(n)]
        if isinstance(params, SamplingParams):
            return [params] * n
        if len(params) != n:
            raise ValueError(f"{len(params)} sampling settings for {n} prompts")
        return list(params)


def _engine_config(max_seq_len, max_gpu_num_blocks, compiled_model, dtype, **extra) -> EngineConfig:
    return EngineConfig(dtype=dtype, max_seq_len=max_seq_len, max_gpu_num_blocks=max_gpu_num_blocks,
                        compiled_model=compiled_model, **extra)


class _TextMixin:
    tokenizer = None

    def load_tokenizer(self, tokenizer_path):
        """A Hugging Face tokenizer for the text entry points (lite_llama/generate.py:78-85); the
        token-id entry points need none."""
        if tokenizer_path is None:
            return None
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(tokenizer_path, use_fast=True)

    def _need_tokenizer(self):
        if self.tokenizer is None:
            raise RuntimeError("text entry points need tokenizer_path; use generate() with token ids otherwise")
        return self.tokenizer


class GenerateText(_TextMixin):
    """lite_llama/generate.py:47-206 with a continuous-batching engine underneath."""

    def __init__(self, checkpoints_dir: str, tokenizer_path: Optional[str] = None, max_seq_len: int = 1024,
                 max_gpu_num_blocks=None, load_model: bool = True, triton_weight: bool = True,
                 compiled_model: bool = False, device: str = "cuda", dtype="bfloat16", **engine_options):
        dev = "cuda:0" if device == "cuda" else device
        self.llm = LLM(checkpoints_dir, _engine_config(max_seq_len, max_gpu_num_blocks, compiled_model, dtype,
                                                       **engine_options), device=dev)
        self.model_config = self.llm.engine.model_config
        self.tokenizer = self.load_tokenizer(tokenizer_path)
        self.device = dev

    def generate(self, prompt_tokens: List[List[int]], max_gen_len: Optional[int], temperature: float = 0.6,
                 top_p: float = 0.9, echo: bool = False, logprobs: bool = False):
        """Token ids generated for each prompt, cut before the first end-of-sequence token
        (lite_llama/generate.py:192-204); with ``echo`` the prompt is put in front.  With ``logprobs``
        the result is (tokens, log-probabilities of the generated tokens), as in
        lite_llama/generete_with_probs.py:87-96,154-165."""
        params = SamplingParams(temperature=temperature, top_p=top_p, max_gen_len=max_gen_len, logprobs=logprobs)
        reqs = [self.llm.add_request(p, params) for p in prompt_tokens]
        for _ in self.llm.run():
            pass
        self.llm.engine.check_device_status()
        eos = self.llm.engine.eos_token_ids
        toks = [_trim(p, r.output, echo, eos) for p, r in zip(prompt_tokens, reqs)]
        if not logprobs:
            return toks
        kept = [len(_trim(p, r.output, False, eos)) for p, r in zip(prompt_tokens, reqs)]
        return toks, [r.logprobs[:n] for r, n in zip(reqs, kept)]

    def text_completion(self, prompts: List[str], temperature: float = 0.6, top_p: float = 0.9,
                        max_gen_len: Optional[int] = None, echo: bool = False) -> List[str]:
        tok = self._need_tokenizer()
        ids = [tok.encode(p, add_special_tokens=True) for p in prompts]
        outs = self.generate(ids, max_gen_len, temperature, top_p, echo)
        return [tok.decode(o, skip_special_tokens=True) for o in outs]


class GenerateStreamText(_TextMixin):
    """lite_llama/generate_stream.py:51-216: the same, yielding as tokens arrive."""

    def __init__(self, checkpoints_dir: str, tokenizer_path: Optional[str] = None, max_gpu_num_blocks=None,
                 max_seq_len: int = 1024, load_model: bool = True, triton_weight: bool = True,
                 compiled_model: bool = False, device: str = "cuda", dtype="bfloat16", **engine_options):
        dev = "cuda:0" if device == "cuda" else device
        self.llm = LLM(checkpoints_dir, _engine_config(max_seq_len, max_gpu_num_blocks, compiled_model, dtype,
                                                       **engine_options), device=dev)
        self.model_config = self.llm.engine.model_config
        self.tokenizer = self.load_tokenizer(tokenizer_path)
        self.device = dev

    def generate_stream(self, prompt_tokens: List[List[int]], max_gen_len: Optional[int],
                        temperature: float = 0.6, top_p: float = 0.9, echo: bool = False
                        ) -> Generator[List[List[int]], None, None]:
        """Yields, per step, the new token ids of every prompt (an empty list where a prompt got
        none); with ``echo`` the first yield of a prompt starts with the prompt itself."""
        params = SamplingParams(temperature=temperature, top_p=top_p, max_gen_len=max_gen_len)
        eos = set(self.llm.engine.eos_token_ids)
        pending_echo = [echo] * len(prompt_tokens)
        for events in self.llm.generate_stream(prompt_tokens, params):
            batch: List[List[int]] = [[] for _ in prompt_tokens]
            for i, toks, done in events:
                new = [t for t in toks if t not in eos]
                if pending_echo[i] and (new or done):
                    new = list(prompt_tokens[i]) + new
                    pending_echo[i] = False
                batch[i] = new
            yield batch

    def text_completion_stream(self, prompts: List[str], temperature: float = 0.6, top_p: float = 0.9,
                               max_gen_len: Optional[int] = None, echo: bool = False):
        """Yields the list of {'generation': text so far, 'tokens': ids so far} after every step
        (lite_llama/generate_stream.py:190-216)."""
        tok = self._need_tokenizer()
        ids = [tok.encode(p, add_special_tokens=True) for p in prompts]
        completions = [{"generation": "", "tokens": []} for _ in prompts]
        for batch in self.generate_stream(ids, max_gen_len, temperature, top_p, echo):
            for i, new in enumerate(batch):
                if new:
                    completions[i]["tokens"] = completions[i]["tokens"] + new
                    completions[i]["generation"] = tok.decode(completions[i]["tokens"], skip_special_tokens=True)
            yield [dict(c) for c in completions]


def _trim(prompt: Sequence[int], output: Sequence[int], echo: bool, eos: Iterable[int]) -> List[int]:
    eos = set(eos)
    cut = list(output)
    for i, t in enumerate(cut):
        if t in eos:
            cut = cut[:i]
            break
    return (list(prompt) + cut) if echo else cut
