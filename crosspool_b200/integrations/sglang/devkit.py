"""Debug-only observers and offline request facts for a serving engine that hosts Instance ranks.

Two tools, both opt-in and both outside the serving hot path:

* ``GraphObserver`` wraps the CUDA-graph ``capture`` / ``execute`` methods of an engine's decode and prefill graph
  runners and appends one JSON line per transition (``capture_begin``, ``capture_end``, ``capture_error``, ``execute_*``)
  to a per-process file ``xpool.graph-observer.<pid>.jsonl`` in ``debug.graph_observer.outdir``. A failure to record
  never disturbs the engine. Reference: src/xpool/integrations/sglang/devkit/graph_observer.py:41-162 (the event record
  is ``SglangGraphEvent`` of devkit/__init__.py).
* ``RequestLimits`` / ``LocalModelMetadata`` state, before any server runs, which (input, output) lengths the engine
  will accept without shortening: input strictly below ``max_req_input_len``, one token reserved below the request
  bound, one free page beyond the paged request when the KV ceiling is known. The load generator uses them to clamp
  sampled lengths. Reference: src/xpool/integrations/sglang/devkit/requests.py:15-113.

The runner classes are passed in (the plugin resolves them from the engine's registry, tests pass fakes); this
repository's own engine is observed through the same wrapper (``observe_engine``).
"""

from __future__ import annotations

import functools
import json
import os
import threading
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterable, Mapping

from ...logging import get_logger

GRAPH_EVENT_FIELDS = ("pid", "model_id", "time_ns", "forward_phase", "backend_class", "event")
_OPERATIONS = ("capture", "execute")


class GraphObserver:
    """One per process. ``model_id_of(runner)`` names the model a runner serves (the plugin maps the runner's model path
    through the deployment config); ``backend_of(runner)`` names its attention backend class."""

    def __init__(self, outdir: str | os.PathLike, model_id_of: Callable[[object], str] | None = None,
                 backend_of: Callable[[object], str] | None = None, clock: Callable[[], int] = time.monotonic_ns):
        if not outdir:
            raise RuntimeError("the graph observer needs debug.graph_observer.outdir")
        self.outdir = Path(outdir)
        self._model_id_of = model_id_of or (lambda r: str(getattr(r, "model_id", "")))
        self._backend_of = backend_of or (lambda r: type(getattr(r, "backend", r)).__name__)
        self._clock = clock
        self._write_lock = threading.Lock()
        self._install_lock = threading.Lock()
        self._handle = None
        self.path: Path | None = None
        self._patched: list[tuple[type, str, Callable]] = []
        self.dropped = 0

    # ------------------------------------------------------------------ file
    def open(self) -> Path:
        """Creates the directory and (re)opens this process's event file; a forked child gets a file of its own."""
        with self._install_lock:
            self.outdir.mkdir(parents=True, exist_ok=True)
            want = self.outdir / f"xpool.graph-observer.{os.getpid()}.jsonl"
            if self.path != want or self._handle is None or self._handle.closed:
                if self._handle is not None and not self._handle.closed:
                    self._handle.close()
                self._handle = want.open("a" if self.path == want else "w", encoding="utf-8")
                self.path = want
            return want

    def close(self) -> None:
        with self._install_lock:
            if self._handle is not None and not self._handle.closed:
                self._handle.close()
            self._handle = None

    # ------------------------------------------------------------------ patching
    def install(self, runners: Mapping[str, type], operations: Iterable[str] = _OPERATIONS) -> None:
        """``runners``: forward phase ("decode" / "prefill") -> graph runner class. Wraps each operation the class has;
        installing twice wraps once."""
        self.open()
        with self._install_lock:
            for phase, cls in runners.items():
                if phase not in ("decode", "prefill"):
                    raise ValueError(f"forward phase {phase!r} is neither 'decode' nor 'prefill'")
                for op in operations:
                    own = cls.__dict__.get(op)
                    original = own or getattr(cls, op, None)
                    if original is None:
                        continue
                    if getattr(original, "__xpool_graph_observer__", None) is self:
                        if own is not None:
                            continue                      # already wrapped on this class
                        original = original.__wrapped__   # inherited from an observed base: this class has its own phase
                    setattr(cls, op, self.wrap(phase, op, original))
                    self._patched.append((cls, op, original))

    def uninstall(self) -> None:
        with self._install_lock:
            for cls, op, original in reversed(self._patched):
                setattr(cls, op, original)
            self._patched.clear()
        self.close()

    def wrap(self, phase: str, operation: str, original: Callable) -> Callable:
        observer = self

        @functools.wraps(original)
        def wrapped(runner, *args, **kwargs):
            observer.write(phase, f"{operation}_begin", runner)
            try:
                result = original(runner, *args, **kwargs)
            except BaseException:
                observer.write(phase, f"{operation}_error", runner)
                raise
            observer.write(phase, f"{operation}_end", runner)
            return result

        wrapped.__xpool_graph_observer__ = observer
        return wrapped

    def write(self, phase: str, event: str, runner) -> None:
        try:
            h = self._handle
            if h is None or h.closed:
                return
            line = json.dumps({"pid": os.getpid(), "model_id": self._model_id_of(runner), "time_ns": self._clock(),
                               "forward_phase": phase, "backend_class": self._backend_of(runner), "event": event})
            with self._write_lock:
                h.write(line + "\n")
                h.flush()
        except Exception:     # recording must never disturb the engine
            self.dropped += 1
            get_logger().warning("failed to record a graph observer event", exc_info=True)


def read_graph_events(outdir: str | os.PathLike) -> list[dict]:
    """All processes' events of a directory, ordered by time."""
    events = []
    for p in sorted(Path(outdir).glob("xpool.graph-observer.*.jsonl")):
        for line in p.read_text(encoding="utf-8").splitlines():
            if line.strip():
                events.append(json.loads(line))
    return sorted(events, key=lambda e: e["time_ns"])


def install_from_config(cfg, runners: Mapping[str, type], model_id_of: Callable[[object], str] | None = None
                        ) -> GraphObserver | None:
    """The plugin's entry: installs the observer when ``debug.graph_observer.enable`` is set."""
    if not cfg.debug_graph_observer_enable:
        return None
    obs = GraphObserver(cfg.debug_graph_observer_outdir, model_id_of=model_id_of)
    obs.install(runners)
    return obs


def observe_engine(observer: GraphObserver, engine_cls: type | None = None) -> None:
    """Observes this repository's own attention engine: graph capture (``_capture_decode``) is the capture operation,
    a graph replay (``_replay_decode``) the execute operation of the decode phase."""
    if engine_cls is None:
        from ...engine.atn_engine import AttentionEngine as engine_cls
    observer.open()
    for op, name in (("capture", "_capture_decode"), ("execute", "_replay_decode")):
        original = getattr(engine_cls, name, None)
        if original is None or getattr(original, "__xpool_graph_observer__", None) is observer:
            continue
        setattr(engine_cls, name, observer.wrap("decode", op, original))
        observer._patched.append((engine_cls, name, original))


# ---------------------------------------------------------------------------------------------- request limits
@dataclass(frozen=True)
class RequestLimits:
    """Static acceptance bounds of one engine, independent of how much elastic KV is backed at the moment."""

    context_length: int
    max_req_input_len: int
    max_total_num_tokens: int | None = None
    page_size: int = 1
    dcp_size: int = 1

    def __post_init__(self):
        for name in ("context_length", "max_req_input_len", "page_size", "dcp_size"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")
        if self.max_total_num_tokens is not None and self.max_total_num_tokens <= 0:
            raise ValueError("max_total_num_tokens must be positive")

    @classmethod
    def from_context(cls, context_length: int) -> "RequestLimits":
        """The model-only bounds: the engine keeps six tokens of the context back from the input."""
        return cls(context_length=context_length, max_req_input_len=context_length - 6)

    @classmethod
    def from_server_info(cls, contents: bytes | str, *, context_length: int) -> "RequestLimits":
        """From the engine's ``/server_info`` answer: the first scheduler's start-up limits, not a DP aggregate."""
        info = json.loads(contents)
        try:
            return cls(context_length=context_length, max_req_input_len=int(info["max_req_input_len"]),
                       max_total_num_tokens=int(info["max_total_num_tokens"]), page_size=int(info["page_size"]),
                       dcp_size=int(info.get("dcp_size", 1)))
        except KeyError as e:
            raise ValueError(f"/server_info lacks {e.args[0]!r}") from None

    @classmethod
    def from_engine_config(cls, ecfg, kv_tokens: int | None = None) -> "RequestLimits":
        """The same bounds for this repository's own engine (``EngineConfig``)."""
        return cls(context_length=ecfg.max_seq_len, max_req_input_len=ecfg.max_seq_len - 1, max_total_num_tokens=kv_tokens,
                   page_size=ecfg.page_size)

    def input_budget(self, output_tokens: int) -> int:
        return min(self.max_req_input_len - 1, self.context_length - output_tokens, self.max_req_input_len + 4 - output_tokens)

    def output_budget(self, input_tokens: int) -> int:
        budget = min(self.context_length - input_tokens, self.max_req_input_len + 4 - input_tokens)
        if self.max_total_num_tokens is not None:
            paged_input = -(-input_tokens // self.page_size) * self.page_size
            budget = min(budget, self.max_total_num_tokens * self.dcp_size - paged_input - self.page_size - 1)
        return budget

    def validate_request(self, input_tokens: int, output_tokens: int) -> None:
        if input_tokens > self.input_budget(output_tokens) or output_tokens > self.output_budget(input_tokens):
            raise ValueError(f"input={input_tokens}, output={output_tokens} exceeds the static service limits "
                             f"(context={self.context_length}, input_bound={self.max_req_input_len}, "
                             f"kv_ceiling={self.max_total_num_tokens}, page_size={self.page_size}, dcp_size={self.dcp_size})")

    def clamp(self, input_tokens: int, output_tokens: int) -> tuple[int, int]:
        """The nearest admissible pair: the output is kept, the input shortened first."""
        n_in = max(1, min(input_tokens, self.input_budget(output_tokens)))
        if self.max_total_num_tokens is not None and self.output_budget(n_in) < output_tokens:
            # the KV ceiling binds: the longest page-aligned input that leaves room for the output, a page and a token
            room = self.max_total_num_tokens * self.dcp_size - self.page_size - 1 - output_tokens
            n_in = max(1, min(n_in, room // self.page_size * self.page_size))
        return n_in, max(1, min(output_tokens, self.output_budget(n_in)))


@dataclass(frozen=True)
class LocalModelMetadata:
    """Facts about a local checkpoint resolved once while a workload is prepared: the vocabulary, the request limits,
    the token ids a synthetic prompt may draw from (no special tokens), and the token length of every text prompt."""

    vocab_size: int
    limits: RequestLimits
    admissible_ids: tuple[int, ...]
    text_lengths: dict[str, int] = field(default_factory=dict)

    def __post_init__(self):
        if self.vocab_size <= 0:
            raise ValueError("vocab_size must be positive")
        if any(t < 0 or t >= self.vocab_size for t in self.admissible_ids):
            raise ValueError("admissible token ids exceed the model's vocabulary")

    @classmethod
    def from_config(cls, hf_config: Mapping, *, special_ids: Iterable[int] = (), vocab: Iterable[int] | None = None,
                    text_lengths: Mapping[str, int] | None = None) -> "LocalModelMetadata":
        """From a parsed ``config.json`` (and, when a tokenizer was read, its ids): no files are opened here."""
        vocab_size = int(hf_config["vocab_size"])
        context = int(hf_config.get("max_position_embeddings") or hf_config.get("n_positions") or 0)
        if context <= 0:
            raise ValueError("the model config names no context length")
        special = set(special_ids)
        ids = range(vocab_size) if vocab is None else vocab
        admissible = tuple(sorted({i for i in ids if 0 <= i < vocab_size and i not in special}))
        for pid, n in (text_lengths or {}).items():
            if n >= context:
                raise ValueError(f"prompt {pid!r} exceeds the model's input limit")
        return cls(vocab_size, RequestLimits.from_context(context), admissible, dict(text_lengths or {}))

    @classmethod
    def from_checkpoint(cls, path: str | os.PathLike, *, text_prompts: Mapping[str, str] | None = None) -> "LocalModelMetadata":
        """Local files only. The tokenizer is optional: a checkpoint without one admits every id below the vocabulary
        size and accepts no text prompts."""
        path = Path(path)
        cfg = json.loads((path / "config.json").read_text(encoding="utf-8"))
        cfg = cfg.get("text_config") or cfg
        tokenizer = None
        if any((path / f).exists() for f in ("tokenizer.json", "tokenizer.model", "vocab.json")):
            from transformers import AutoTokenizer

            tokenizer = AutoTokenizer.from_pretrained(str(path), local_files_only=True)
        if tokenizer is None:
            if text_prompts:
                raise ValueError("text prompts need the checkpoint's tokenizer")
            return cls.from_config(cfg)
        vocab_size = int(cfg["vocab_size"])
        lengths = {}
        for pid, text in (text_prompts or {}).items():
            tokens = tokenizer.encode(text)
            if any(t < 0 or t >= vocab_size for t in tokens):
                raise ValueError(f"prompt {pid!r} contains ids outside the model's vocabulary")
            lengths[pid] = len(tokens)
        return cls.from_config(cfg, special_ids=tokenizer.all_special_ids, vocab=tokenizer.get_vocab().values(),
                               text_lengths=lengths)
