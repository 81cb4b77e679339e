"""The generator: the package's Python entry point, in the reference's manner.

    fg = Fastgen.build(HfLoader(model_dir), GenArgs(...), tp_mesh=None,
                       device=torch.device("cuda:0"))
    q = queue.Queue()
    q.put(Packet(thread_id=0, tokens=[...], temperature=0.8, max_gen=24))
    q.put(None)
    for pkt in fg.generate(q):
        ...
    fg.destroy()

Names and meanings of ``GenArgs``, ``Packet``, ``Fastgen.build/generate/destroy``
follow fastgen/generate.py:30-76, 139-173, 405-425.  Options of the reference
that belong to features outside this engine (host cache, fp8, tensor
parallelism) are not present; ``tp_mesh`` must be ``None``.
"""

from __future__ import annotations

import logging
import os
import queue
import tempfile
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Generator, List, Optional, Union

import torch

from ..config import load_model_args, read_config
from ..csrc.ops import describe_status
from ..sampling import Sampler
from ..utils.misc import hashints
from .model import Model
from .scheduler import Request, Scheduler
from .step import Engine, StepEntry
from .tune import mem_params

logger = logging.getLogger("fastgen_b200")


@dataclass
class GenArgs:
    use_sampling: bool = True
    temperature: float = 0.7
    top_p: float = 0.9
    logprobs: bool = False

    max_batch: int = 256
    max_seq: int = -1  # total cache tokens; negative: from the memory budget
    max_gen: Optional[int] = None

    cache_block: int = 64  # tokens per cache page
    num_cuda_graphs: int = 16

    max_prefill: int = 8192  # tokens per step, prompt portions and decoded tokens together
    min_prefill: int = 2048  # newly admitted prompts with fewer tokens than this together ...
    min_prefill_batch: int = 1  # ... and fewer requests than this wait while others decode
    prefill_gb: float = 0.5  # used by the memory budget
    gpu_gb: float = 20  # ditto

    sync_freq: int = 10
    seed: int = 777


@dataclass
class Packet:
    thread_id: Any
    "An arbitrary identifier to link inputs to outputs."
    tokens: List[int] = field(default_factory=list)
    "The prompt if used as input, or else the generation output."
    temperature: Optional[float] = None
    "An optional per-generation temperature setting."
    logprobs: Optional[List[float]] = None
    "Logprobs of the output tokens; only when ``GenArgs.logprobs`` is set."
    max_gen: Optional[int] = None
    "The maximum number of tokens to generate."
    error: Optional[str] = None
    "Set on an output packet whose request could not be served."


class HfLoader:
    """A model folder: ``config.json``, safetensors and (optionally) a tokenizer."""

    def __init__(self, model: Union[str, Path]) -> None:
        self.directory = Path(model)
        read_config(self.directory)  # fails early with a clear error

    def load_model_args(self):
        return load_model_args(self.directory)

    def load_tokenizer(self):
        from ..utils.tokenizer import HfTokenizer

        return HfTokenizer(self.directory)

    def has_tokenizer(self) -> bool:
        return (self.directory / "tokenizer.json").is_file()

    def load(self, dtype: torch.dtype, device) -> Model:
        return Model.load(self.directory, dtype, device)


class Fastgen:
    @staticmethod
    def build(loader: HfLoader, gen_args: GenArgs, tp_mesh=None,
              device: Union[str, torch.device] = "cuda:0",
              dtype: torch.dtype = torch.bfloat16, profile_sig: Optional[int] = None) -> "Fastgen":
        """``profile_sig``: a signal number (the reference's default is SIGUSR2,
        generate.py:145,166-172) on which a trace of the next scheduler iterations is
        written, see ``request_profile``; ``None`` installs no handler."""
        if tp_mesh is not None:
            raise ValueError("this engine runs on one GPU; tp_mesh must be None")
        device = torch.device(device)
        t0 = time.monotonic()
        model = loader.load(dtype, device)
        logger.info("Built and loaded model in %.2fs", time.monotonic() - t0)
        stop_tokens = list(model.args.stop_tokens)
        if loader.has_tokenizer():
            stop_tokens = loader.load_tokenizer().stop_tokens or stop_tokens
        fg = Fastgen(gen_args, model, stop_tokens)
        if profile_sig is not None:
            import signal

            if signal.getsignal(profile_sig) is signal.SIG_DFL:  # never replace somebody's handler
                signal.signal(profile_sig, lambda _signum, _frame: fg.request_profile())
        return fg

    def __init__(self, args: GenArgs, model: Model, stop_tokens) -> None:
        self.gen_args = args
        self.model = model
        self.ops = model.ops
        self.device = model.ops.device
        self.stop_tokens = list(stop_tokens)
        self.generating = False
        block = args.cache_block
        act_bytes = 4 if model.ops.act_dtype == torch.float32 else 2
        self._last_used_gb: Optional[float] = None
        logger.info("Initializing generator")
        self._log_cuda_mem()

        # pages: from max_seq, or from the memory budget (generate.py:206-236)
        per_token = model.cache_bytes_per_token(act_bytes)
        widest = max((getattr(l.ffn.params, "ffn_dim", model.args.dim) for l in model.args.layers))
        mp = mem_params(model.weight_bytes(), per_token, model.args.dim, widest, act_bytes,
                        max(args.prefill_gb, 0.1), args.gpu_gb)
        mp.round_to(block)
        max_seq = args.max_seq
        if max_seq < 0:
            max_seq = mp.cache_tokens
            logger.info("Setting max sequence length to %d", max_seq)
        max_seq = -(-max_seq // block) * block
        if max_seq < block:
            raise RuntimeError("Not enough memory available for the generation caches")
        self.max_seq = max_seq
        self.max_prefill = args.max_prefill if args.max_prefill > 0 else mp.prefill_tokens
        if args.max_prefill <= 0:
            logger.info("Setting max prefill length to %d", self.max_prefill)
        self.max_batch = min(args.max_batch, max_seq // block)
        if self.max_batch < args.max_batch:
            logger.info("Adjusting max batch to %d", self.max_batch)

        self.engine = Engine(
            model, page_size=block, n_pages=max_seq // block, max_requests=self.max_batch,
            max_length=min(model.args.max_positions, max_seq), num_cuda_graphs=args.num_cuda_graphs,
            max_step_tokens=self.max_prefill,
        )
        logger.info("Cache bytes per token: %d", per_token)
        logger.info("Allocated kv cache: %d pages of %d tokens", max_seq // block, block)
        self._log_cuda_mem()
        self.sampler = Sampler(
            self.ops, model.args.vocab_size, self.max_batch, use_sampling=args.use_sampling,
            top_p=args.top_p, seed=args.seed, logprobs=args.logprobs,
        )
        self.scheduler = Scheduler(
            self.engine.cache, self.max_batch, self.max_prefill, self.stop_tokens, args.max_gen,
            min_prefill=args.min_prefill, min_prefill_batch=args.min_prefill_batch,
        )
        self.steps = 0
        # per step: host times, decoded and prompt tokens, bytes copied, cached positions read
        # (kv_tokens) and (query, key) pairs of its attention (key_pairs)
        self.step_log: List[dict] = []
        # a trace on request (generate.py:187-196, 364-403): FG_PROFILE_ITERS scheduler iterations
        # after ``request_profile()``, written as a chrome trace into FG_PROFILE_DIR
        self.profile_iters = int(os.environ.get("FG_PROFILE_ITERS", "8"))
        self.profile_dir = os.environ.get("FG_PROFILE_DIR", tempfile.gettempdir())
        self.profile_state = "inactive"  # -> "requested" -> "active" -> "inactive"
        self.profile_left = 0
        self.profiler = None
        self.last_profile: Optional[str] = None  # path of the trace written last
        if self.engine.graphs is not None:
            # as the reference does when it is built (generate.py:300-347): no step waits for a capture
            self.engine.graphs.capture_all()
            logger.info("Created %d decoding graphs", len(self.engine.graphs.buckets))
            self._log_cuda_mem()
        logger.info("Done initializing")

    def _log_cuda_mem(self) -> None:
        used_gb = torch.cuda.memory_allocated(self.device) / 1e9
        if self._last_used_gb is None:
            logger.info("GPU memory: %.3fGB", used_gb)
        else:
            logger.info("GPU memory: %.3fGB (%+.3fGB)", used_gb, used_gb - self._last_used_gb)
        self._last_used_gb = used_gb

    def request_profile(self) -> None:
        """Ask for a trace (CPU and CUDA activity) of the next ``FG_PROFILE_ITERS`` iterations
        of the scheduler loop; it is written to ``FG_PROFILE_DIR`` when they are over."""
        if self.profile_state == "inactive":
            logger.info("Requesting profiling trace...")
            self.profile_state = "requested"

    def _profile_tick(self) -> None:
        """Once per iteration of the scheduler loop."""
        if self.profile_state == "requested":
            from torch.profiler import ProfilerActivity, profile

            self.profiler = profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], with_stack=True)
            self.profiler.__enter__()
            self.profile_left = self.profile_iters
            self.profile_state = "active"
        elif self.profile_state == "active":
            self.profile_left -= 1
            if self.profile_left <= 0:
                self._profile_stop()

    def _profile_stop(self) -> None:
        if self.profile_state != "active":
            return
        self.profile_state = "inactive"
        prof, self.profiler = self.profiler, None
        try:
            prof.__exit__(None, None, None)
            stamp = time.strftime("%H%M%S") + f".{int(time.time() * 1e6) % 1_000_000:06d}"
            path = os.path.join(self.profile_dir, f"fastgen_b200_{os.getpid()}_{stamp}.json.gz")
            prof.export_chrome_trace(path)
            self.last_profile = path
            logger.info("Profile chrome trace exported to %s", path)
        except Exception as e:  # noqa: BLE001 - a failed trace must not end generation
            logger.warning("Error while exporting profile trace: %r", e)

    def destroy(self) -> None:
        """Free what the generator holds on the device."""
        self._profile_stop()
        self.engine = None
        self.scheduler = None
        self.sampler = None

    # -- the loop ----------------------------------------------------------------
    def _packet(self, req: Request) -> Packet:
        return Packet(
            thread_id=req.thread_id,
            tokens=list(req.generated),
            temperature=req.temperature,
            logprobs=list(req.logprobs) if self.gen_args.logprobs else None,
            max_gen=req.max_gen,
            error=req.error,
        )

    def _pull(self, q: "queue.Queue[Optional[Packet]]", eoq: bool) -> bool:
        """Move packets from the queue to the scheduler; block only when idle."""
        while not eoq:
            try:
                pkt = q.get(block=not self.scheduler.has_work())
            except queue.Empty:
                break
            if pkt is None:
                self.scheduler.input_ended = True
                return True
            # generate.py:790: a per-request temperature of 0 falls back to the default
            temp = pkt.temperature or self.gen_args.temperature
            if not self.gen_args.use_sampling:
                temp = 0.0
            self.scheduler.add(pkt.thread_id, pkt.tokens, temp, pkt.max_gen)
            if logger.isEnabledFor(logging.DEBUG):
                # the reference keeps this hash on every lane (generate.py:112)
                logger.debug("request %s: %d prompt tokens, hash %d", pkt.thread_id, len(pkt.tokens),
                             hashints(pkt.tokens))
            if len(self.scheduler.waiting) >= 2 * self.max_batch:
                break
        return eoq

    def generate(self, q: "queue.Queue[Optional[Packet]]") -> Generator[Packet, None, None]:
        """Read prompts from the queue and yield a completion (or an error) for
        each; outputs may come in another order than inputs.  ``None`` in the
        queue ends the input; what is in flight is completed."""
        assert not self.generating, "multiple generators cannot run concurrently"
        self.generating = True
        try:
            yield from self._generate(q)
        finally:
            self.generating = False

    def _decode_run(self, n_steps: int):
        """``n_steps`` decode steps of all running requests; the sampled tokens feed the
        next step on the device and come to the host once, at the end."""
        sched, engine = self.scheduler, self.engine
        reqs = list(sched.running)
        handles = [engine.cache.get(id(r)) for r in reqs]
        slots = [h.slot for h in handles]
        temps = [r.temperature for r in reqs]
        keys = [r.key for r in reqs]
        t_start = time.perf_counter()
        engine.cache.flush_tables()
        tokens = [r.generated[-1] if r.generated else r.prompt[-1] for r in reqs]
        outs, lps = [], []
        for k in range(n_steps):
            logits = engine.graphs.run(tokens, [h.length + k for h in handles], slots)
            out, lp = self.sampler.sample(logits, temps, keys, [len(r) + k for r in reqs])
            outs.append(out)
            lps.append(lp)
            tokens = out  # stays on the device
        sampled = torch.stack(outs).tolist()  # the run's one device-to-host read
        logprobs = torch.stack(lps).tolist() if lps[0] is not None else None
        # the last entry of a step's row is the device status word after that step
        word = 0
        for row in sampled:
            word |= row.pop()
        self.steps += n_steps
        t_end = time.perf_counter()
        lengths = sum(h.length for h in handles)
        for k in range(n_steps):
            self.step_log.append(dict(
                t_start=t_start + (t_end - t_start) * k / n_steps,
                t_end=t_start + (t_end - t_start) * (k + 1) / n_steps,
                decode_tokens=len(reqs), prompt_tokens=0,
                h2d_bytes=engine.graphs.last_h2d_bytes, d2h_bytes=4 * (len(reqs) + 1),
                kv_tokens=lengths + (k + 1) * len(reqs), key_pairs=lengths + (k + 1) * len(reqs),
            ))
        if word:
            yield from self._fail_step(reqs, word)
            return
        for req in sched.commit_decode_run(reqs, sampled, logprobs):
            yield self._packet(req)

    def _fail_step(self, reqs, word: int):
        """A kernel of the step recorded a fault in the status word (a missing page, a token
        outside the vocabulary, a wait that ran out) instead of performing a bad access: what
        the step computed is void.  Its requests end with ``Packet.error``; the word is
        cleared, the others go on."""
        message = describe_status(word)
        logger.error("%s; ending %d request(s) of the step", message, len(reqs))
        self.ops.clear_status()
        for req in self.scheduler.fail(reqs, message):
            yield self._packet(req)

    @torch.inference_mode()
    def _generate(self, q):
        sched = self.scheduler
        eoq = False
        while not eoq or sched.has_work() or sched.finished:
            if self.profile_state != "inactive":
                self._profile_tick()
            eoq = self._pull(q, eoq)
            for req in sched.take_finished():
                yield self._packet(req)
            # several decode steps without a host round trip, when nothing else is to be decided
            n_run = 1
            if self.engine.graphs is not None and q.empty():
                n_run = sched.plan_decode_run(self.gen_args.sync_freq)
            if n_run > 1:
                yield from self._decode_run(n_run)
                continue
            plan = sched.plan()
            if logger.isEnabledFor(logging.INFO):
                logger.info("%d active requests", len(sched.running))
                n_prompt = sum(len(e.tokens) for e in plan if not (len(e.tokens) == 1 and e.request.generated))
                if n_prompt:
                    logger.info("Prefilling %d tokens", n_prompt)
            if not plan:
                if sched.has_work():
                    raise RuntimeError("the scheduler made no progress")  # cannot happen: see Scheduler.add
                continue
            entries = [
                StepEntry(id(e.request), e.tokens, [len(e.tokens) - 1] if e.samples else [])
                for e in plan
            ]
            t_start = time.perf_counter()
            # cached positions the step reads, and (query, key) pairs its attention forms
            kv_tokens = key_pairs = 0
            for e in plan:
                before, n = self.engine.cache.get(id(e.request)).length, len(e.tokens)
                kv_tokens += before + n
                key_pairs += n * before + n * (n + 1) // 2
            logits = self.engine.step_reserved(entries)
            self.steps += 1
            sampling = [e for e in plan if e.samples]
            tokens: List[int] = []
            logprobs = None
            word = 0
            if sampling:
                out, lp = self.sampler.sample(
                    logits,
                    [e.request.temperature for e in sampling],
                    [e.request.key for e in sampling],
                    [len(e.request) for e in sampling],
                )
                tokens = out.tolist()  # the step's one device-to-host read
                word = tokens.pop()  # the device status word rides along
                logprobs = lp.tolist() if lp is not None else None
            n_decode = sum(1 for e in plan if len(e.tokens) == 1 and e.samples and e.request.generated)
            self.step_log.append(dict(
                t_start=t_start, t_end=time.perf_counter(), decode_tokens=n_decode,
                prompt_tokens=sum(len(e.tokens) for e in plan) - n_decode,
                h2d_bytes=self.engine.last_h2d_bytes, d2h_bytes=4 * (len(tokens) + 1) if sampling else 0,
                kv_tokens=kv_tokens, key_pairs=key_pairs,
            ))
            if len(self.step_log) > 100_000:
                del self.step_log[:50_000]
            if word:
                yield from self._fail_step([e.request for e in plan], word)
                continue
            for req in sched.commit(plan, tokens, logprobs):
                yield self._packet(req)
