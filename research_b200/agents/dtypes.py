"""Core data types of the agent runtime: messages, tool calls, trajectories, environments,
endpoints, run configuration, scores (surface of rollouts/dtypes.py:192-1487, condensed).

Everything is a plain dataclass that round-trips through JSON; ``Trajectory`` is the unit
that rollout generation turns into training ``Sample``s, and ``Choice.token_ids`` /
``Choice.logprobs`` carry the engine's exact tokens so training never re-tokenises text
(the "TI/TO" discipline of rollouts/docs/design/tito_correctness_testing.md).
"""

from __future__ import annotations

import hashlib
import json
import time
from dataclasses import asdict, dataclass, field, fields, is_dataclass
from enum import Enum
from pathlib import Path
from typing import Any, Awaitable, Callable, Protocol, runtime_checkable


def parse_streaming_json(partial: str) -> dict[str, Any]:
    """Best-effort reading of a JSON object that is still being streamed (tool-call arguments arrive in pieces): what is
    complete so far, with open strings, arrays and objects closed. ``'{"a": 1, "b":'`` -> ``{"a": 1}``;
    ``'{"path": "src/ma'`` -> ``{"path": "src/ma"}``; anything that is not (yet) an object -> ``{}``."""
    import json

    s = partial.strip()
    if not s.startswith("{"):
        return {}
    try:
        v = json.loads(s)
        return v if isinstance(v, dict) else {}
    except ValueError:
        pass
    closer = {"{": "}", "[": "]"}
    stack: list[str] = []
    cuts: list[tuple[int, tuple[str, ...]]] = []         # places where cutting leaves only complete members
    in_str = esc = False
    for i, ch in enumerate(s):
        if in_str:
            if esc:
                esc = False
            elif ch == "\\":
                esc = True
            elif ch == '"':
                in_str = False
            continue
        if ch == '"':
            in_str = True
        elif ch in "{[":
            stack.append(ch)
            cuts.append((i + 1, tuple(stack)))
        elif ch in "}]" and stack:
            stack.pop()
            cuts.append((i + 1, tuple(stack)))
        elif ch == ",":
            cuts.append((i, tuple(stack)))
    tail = s[:-1] if esc else s                                  # a dangling backslash cannot be closed
    attempts = [(tail + ('"' if in_str else ""), tuple(stack))] + [(s[:pos], st) for pos, st in reversed(cuts[-12:])]
    for text, st in attempts:
        try:
            v = json.loads(text + "".join(closer[c] for c in reversed(st)))
            return v if isinstance(v, dict) else {}
        except ValueError:
            continue
    return {}


# ------------------------------------------------------------------------------ streaming events
@dataclass(frozen=True)
class StreamEvent:
    type: str = "event"
    timestamp: float = field(default_factory=time.time)


@dataclass(frozen=True)
class LLMCallStart(StreamEvent):
    """A request is about to be sent (front ends start their spinner here, before the first byte comes back)."""
    type: str = "llm_call_start"


@dataclass(frozen=True)
class StreamStart(StreamEvent):
    type: str = "start"


@dataclass(frozen=True)
class TextStart(StreamEvent):
    content_index: int = 0
    type: str = "text_start"


@dataclass(frozen=True)
class TextEnd(StreamEvent):
    content_index: int = 0
    content: str = ""                    # the block's complete text
    type: str = "text_end"


@dataclass(frozen=True)
class ThinkingStart(StreamEvent):
    content_index: int = 0
    type: str = "thinking_start"


@dataclass(frozen=True)
class ThinkingEnd(StreamEvent):
    content_index: int = 0
    content: str = ""
    type: str = "thinking_end"


@dataclass(frozen=True)
class ToolCallDelta(StreamEvent):
    """A piece of a tool call's arguments; ``partial_args`` is what ``parse_streaming_json`` makes of everything so far."""
    tool_call_id: str = ""
    delta: str = ""
    partial_args: dict[str, Any] = field(default_factory=dict)
    type: str = "toolcall_delta"


@dataclass(frozen=True)
class ToolCallError(StreamEvent):
    """The model's arguments for a tool call were not valid JSON."""
    tool_call_id: str = ""
    tool_name: str = ""
    error: str = ""
    raw_arguments: str = ""
    type: str = "toolcall_error"


@dataclass(frozen=True)
class ToolExecutionStart(StreamEvent):
    tool_call_id: str = ""
    tool_name: str = ""
    type: str = "tool_execution_start"


@dataclass(frozen=True)
class TextDelta(StreamEvent):
    delta: str = ""
    type: str = "text_delta"


@dataclass(frozen=True)
class ThinkingDelta(StreamEvent):
    delta: str = ""
    type: str = "thinking_delta"


@dataclass(frozen=True)
class ToolCallStart(StreamEvent):
    tool_call_id: str = ""
    name: str = ""
    type: str = "tool_call_start"


@dataclass(frozen=True)
class ToolCallEnd(StreamEvent):
    tool_call_id: str = ""
    name: str = ""
    args: dict[str, Any] = field(default_factory=dict)
    type: str = "tool_call_end"


@dataclass(frozen=True)
class ToolResultReceived(StreamEvent):
    tool_call_id: str = ""
    content: str = ""
    is_error: bool = False
    details: dict[str, Any] = field(default_factory=dict)       # the tool's own extras (an edit's diff, ...) for display
    type: str = "tool_result"


@dataclass(frozen=True)
class StreamDone(StreamEvent):
    stop_reason: str = "stop"
    type: str = "done"


@dataclass(frozen=True)
class StreamError(StreamEvent):
    error: str = ""
    type: str = "error"


# ------------------------------------------------------------------------------ content
@dataclass(frozen=True)
class TextContent:
    text: str
    type: str = "text"


@dataclass(frozen=True)
class ThinkingContent:
    thinking: str
    signature: str | None = None
    type: str = "thinking"


@dataclass(frozen=True)
class ImageContent:
    data: str
    mime_type: str = "image/png"
    type: str = "image"


@dataclass(frozen=True)
class ToolCall:
    id: str
    name: str
    args: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ToolCallContent:
    id: str
    name: str
    arguments: dict[str, Any] = field(default_factory=dict)
    type: str = "tool_call"


ContentBlock = TextContent | ThinkingContent | ImageContent | ToolCallContent


def _block_from_dict(d: dict) -> ContentBlock:
    t = d.get("type", "text")
    if t == "thinking":
        return ThinkingContent(d.get("thinking", ""), d.get("signature"))
    if t == "image":
        return ImageContent(d.get("data", ""), d.get("mime_type", "image/png"))
    if t == "tool_call":
        return ToolCallContent(d["id"], d["name"], d.get("arguments", {}))
    return TextContent(d.get("text", ""))


@dataclass(frozen=True)
class Message:
    role: str                                   # system | user | assistant | tool
    content: str | list[ContentBlock] | None = None
    tool_calls: tuple[ToolCall, ...] = ()
    tool_call_id: str | None = None
    name: str | None = None
    timestamp: float = field(default_factory=time.time)
    metadata: dict[str, Any] = field(default_factory=dict)

    def text(self) -> str:
        if self.content is None:
            return ""
        if isinstance(self.content, str):
            return self.content
        return "".join(b.text for b in self.content if isinstance(b, TextContent))

    def get_tool_calls(self) -> list[ToolCall]:
        calls = list(self.tool_calls)
        if isinstance(self.content, list):
            calls += [ToolCall(b.id, b.name, dict(b.arguments)) for b in self.content if isinstance(b, ToolCallContent)]
        return calls

    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {"role": self.role, "timestamp": self.timestamp}
        if isinstance(self.content, list):
            d["content"] = [asdict(b) for b in self.content]
        else:
            d["content"] = self.content
        if self.tool_calls:
            d["tool_calls"] = [asdict(t) for t in self.tool_calls]
        if self.tool_call_id:
            d["tool_call_id"] = self.tool_call_id
        if self.name:
            d["name"] = self.name
        if self.metadata:
            d["metadata"] = self.metadata
        return d

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "Message":
        content = d.get("content")
        if isinstance(content, list):
            content = [_block_from_dict(b) for b in content]
        return Message(role=d["role"], content=content,
                       tool_calls=tuple(ToolCall(t["id"], t["name"], t.get("args", {})) for t in d.get("tool_calls", [])),
                       tool_call_id=d.get("tool_call_id"), name=d.get("name"), timestamp=d.get("timestamp", 0.0),
                       metadata=d.get("metadata", {}))


# ------------------------------------------------------------------------------ usage / completion
@dataclass(frozen=True)
class Cost:
    input: float = 0.0
    output: float = 0.0
    cache_read: float = 0.0
    cache_write: float = 0.0

    @property
    def total(self) -> float:
        return self.input + self.output + self.cache_read + self.cache_write


@dataclass(frozen=True)
class Usage:
    input_tokens: int = 0
    output_tokens: int = 0
    reasoning_tokens: int = 0
    cache_read_tokens: int = 0
    cache_write_tokens: int = 0
    cost: Cost = field(default_factory=Cost)

    @property
    def total_tokens(self) -> int:
        return self.input_tokens + self.output_tokens

    def __add__(self, o: "Usage") -> "Usage":
        return Usage(self.input_tokens + o.input_tokens, self.output_tokens + o.output_tokens,
                     self.reasoning_tokens + o.reasoning_tokens, self.cache_read_tokens + o.cache_read_tokens,
                     self.cache_write_tokens + o.cache_write_tokens,
                     Cost(self.cost.input + o.cost.input, self.cost.output + o.cost.output,
                          self.cost.cache_read + o.cost.cache_read, self.cost.cache_write + o.cost.cache_write))


@dataclass(frozen=True)
class Logprob:
    token: str
    logprob: float
    token_id: int | None = None
    top_logprobs: tuple[tuple[str, float], ...] = ()


@dataclass(frozen=True)
class Logprobs:
    content: tuple[Logprob, ...] = ()


@dataclass(frozen=True)
class Choice:
    index: int
    message: Message
    finish_reason: str = "stop"
    logprobs: Logprobs | None = None
    token_ids: tuple[int, ...] | None = None        # exact generated token ids (TI/TO)
    prompt_token_ids: tuple[int, ...] | None = None


@dataclass(frozen=True)
class ChatCompletion:
    id: str
    model: str
    choices: tuple[Choice, ...]
    usage: Usage = field(default_factory=Usage)
    created: float = field(default_factory=time.time)
    weight_version: int | None = None


# ------------------------------------------------------------------------------ trajectory
@dataclass(frozen=True)
class Trajectory:
    messages: tuple[Message, ...] = ()
    completions: tuple[ChatCompletion, ...] = ()
    rewards: float = 0.0
    metadata: dict[str, Any] = field(default_factory=dict)

    def append(self, *msgs: Message) -> "Trajectory":
        return Trajectory(self.messages + tuple(msgs), self.completions, self.rewards, self.metadata)

    def with_completion(self, c: ChatCompletion) -> "Trajectory":
        return Trajectory(self.messages, self.completions + (c,), self.rewards, self.metadata)

    def to_dict(self) -> dict[str, Any]:
        return {"messages": [m.to_dict() for m in self.messages], "rewards": self.rewards, "metadata": self.metadata,
                "completions": [{"id": c.id, "model": c.model, "weight_version": c.weight_version,
                                 "usage": asdict(c.usage),
                                 "choices": [{"index": ch.index, "finish_reason": ch.finish_reason,
                                              "message": ch.message.to_dict(),
                                              "token_ids": list(ch.token_ids) if ch.token_ids is not None else None,
                                              "prompt_token_ids": list(ch.prompt_token_ids) if ch.prompt_token_ids is not None else None,
                                              "logprobs": [lp.logprob for lp in ch.logprobs.content] if ch.logprobs else None}
                                             for ch in c.choices]} for c in self.completions]}

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "Trajectory":
        comps = []
        for c in d.get("completions", []):
            chs = []
            for ch in c.get("choices", []):
                lps = ch.get("logprobs")
                chs.append(Choice(ch["index"], Message.from_dict(ch["message"]), ch.get("finish_reason", "stop"),
                                  Logprobs(tuple(Logprob("", float(v)) for v in lps)) if lps is not None else None,
                                  tuple(ch["token_ids"]) if ch.get("token_ids") is not None else None,
                                  tuple(ch["prompt_token_ids"]) if ch.get("prompt_token_ids") is not None else None))
            u = c.get("usage", {})
            usage = Usage(**{k: v for k, v in u.items() if k != "cost"}, cost=Cost(**u.get("cost", {}))) if u else Usage()
            comps.append(ChatCompletion(c["id"], c["model"], tuple(chs), usage, weight_version=c.get("weight_version")))
        return Trajectory(tuple(Message.from_dict(m) for m in d.get("messages", [])), tuple(comps),
                          d.get("rewards", 0.0), d.get("metadata", {}))

    def to_jsonl(self) -> str:
        return json.dumps(self.to_dict())

    @staticmethod
    def save_jsonl(trajs: list["Trajectory"], path: str | Path) -> None:
        Path(path).parent.mkdir(parents=True, exist_ok=True)
        with open(path, "w") as f:
            for t in trajs:
                f.write(t.to_jsonl() + "\n")

    @staticmethod
    def load_jsonl(path: str | Path) -> list["Trajectory"]:
        with open(path) as f:
            return [Trajectory.from_dict(json.loads(line)) for line in f if line.strip()]

    def hash(self) -> str:
        payload = json.dumps([{k: v for k, v in m.to_dict().items() if k != "timestamp"} for m in self.messages], sort_keys=True)
        return hashlib.sha256(payload.encode()).hexdigest()[:16]


# ------------------------------------------------------------------------------ tools / environment
@dataclass(frozen=True)
class ToolFunctionParameter:
    properties: dict[str, Any] = field(default_factory=dict)
    required: tuple[str, ...] = ()
    type: str = "object"


@dataclass(frozen=True)
class ToolFunction:
    name: str
    description: str
    parameters: ToolFunctionParameter = field(default_factory=ToolFunctionParameter)


@dataclass(frozen=True)
class Tool:
    function: ToolFunction
    type: str = "function"

    def to_openai(self) -> dict[str, Any]:
        p = self.function.parameters
        return {"type": "function", "function": {"name": self.function.name, "description": self.function.description,
                                                 "parameters": {"type": p.type, "properties": p.properties,
                                                                "required": list(p.required)}}}


class SessionStatus(Enum):
    PENDING = "pending"
    COMPLETED = "completed"
    TRUNCATED = "truncated"
    ABORTED = "aborted"


@dataclass(frozen=True)
class TokenInfo:
    """One candidate of a prompt-logprob entry as inference servers report it (``{token id: {logprob, rank, decoded_token}}``)."""
    logprob: float
    rank: int
    decoded_token: str


class StopReason(Enum):
    MAX_TURNS = "max_turns"
    TASK_COMPLETED = "task_completed"
    NO_TOOL_CALLS = "no_tool_calls"
    ABORTED = "aborted"
    ERROR = "error"
    LENGTH = "length"
    USER_ABORT = "user_abort"
    BUDGET_EXCEEDED = "budget_exceeded"


@dataclass(frozen=True)
class ToolResult:
    tool_call_id: str
    content: str = ""
    is_error: bool = False
    error: str | None = None
    stop_reason: StopReason | None = None
    metadata: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class ToolConfirmResult:
    """What a confirmation callback may return instead of a bare bool: whether to run the call, the result to record when
    it does not run, and a message from the user that follows the result (guidance on what to do instead)."""
    proceed: bool
    tool_result: ToolResult | None = None
    user_message: str | None = None


@runtime_checkable
class Environment(Protocol):
    """What an agent acts in: advertises tools, executes tool calls, serialises its state."""

    def get_tools(self) -> list[Tool]: ...
    async def exec_tool(self, tool_call: ToolCall, state: "AgentState", run_config: "RunConfig") -> ToolResult: ...
    def requires_confirmation(self, tool_call: ToolCall) -> bool: ...
    async def serialize(self) -> dict[str, Any]: ...

    @staticmethod
    async def deserialize(data: dict[str, Any]) -> "Environment": ...


@dataclass(frozen=True)
class Endpoint:
    provider: str = "native"                    # native | sglang | vllm | openai | anthropic | google | mock
    model: str = ""
    api_base: str = ""
    api_key: str = ""
    oauth_token: str = ""                       # a subscription log-in's access token; sent as a bearer token instead of the key
    max_tokens: int = 1024
    temperature: float = 1.0
    top_p: float | None = None
    reasoning_effort: str | None = None
    max_retries: int = 3
    timeout: float = 120.0
    extra_params: dict[str, Any] = field(default_factory=dict)
    engine: Any = None                          # in-process InferenceEngine for provider == "native"

    def to_dict(self) -> dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name not in ("engine", "api_key", "oauth_token")}
        return d


@dataclass(frozen=True)
class Actor:
    trajectory: Trajectory
    endpoint: Endpoint
    tools: tuple[Tool, ...] = ()


@dataclass(frozen=True)
class AgentState:
    actor: Actor
    environment: Any = None
    turn_idx: int = 0
    max_turns: int = 10
    stop: StopReason | None = None
    pending_tool_calls: tuple[ToolCall, ...] = ()
    next_tool_idx: int = 0
    session_id: str | None = None
    usage: Usage = field(default_factory=Usage)


@dataclass(frozen=True)
class RunConfig:
    on_chunk: Callable[[StreamEvent], Awaitable[None]] | None = None
    on_input: Callable[[str], Awaitable[str]] | None = None
    confirm_tool: Callable[[ToolCall, AgentState, "RunConfig"], Awaitable["bool | ToolConfirmResult"]] | None = None
    on_step_start: Callable[[AgentState], AgentState] | None = None      # before each model call (e.g. a turns-left warning)
    handle_stop: Callable[[AgentState], AgentState] | None = None
    handle_no_tool: Callable[[AgentState, "RunConfig"], Awaitable[AgentState]] | None = None
    use_tito: bool = False
    tokenizer: Any = None
    suffix_ids: tuple[int, ...] | None = None
    api_limiter: Any = None
    tool_limiter: Any = None
    session_store: Any = None
    session_tags: dict[str, Any] | None = None      # stored with a session this run creates (e.g. its fingerprint)
    cancel_event: Any = None
    show_progress: bool = False


# ------------------------------------------------------------------------------ scores / evaluation
@dataclass(frozen=True)
class Metric:
    name: str
    value: float
    weight: float = 0.0                          # weight 0 = tracked only, not part of the reward
    metadata: dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class Score:
    metrics: tuple[Metric, ...] = ()

    @property
    def reward(self) -> float:
        tw = sum(m.weight for m in self.metrics)
        if tw == 0:
            return 0.0
        return sum(m.value * m.weight for m in self.metrics) / tw

    def to_dict(self) -> dict[str, Any]:
        return {"reward": self.reward, "metrics": [asdict(m) for m in self.metrics]}


@dataclass(frozen=True)
class EvalConfig:
    endpoint: Endpoint
    score_fn: Callable[..., Any]
    environment_factory: Callable[..., Any] | None = None
    prepare_messages: Callable[[dict[str, Any]], list[Message]] | None = None
    max_turns: int = 10
    max_samples: int | None = None
    max_concurrent: int = 8
    n_retries: int = 2
    retry_delays: tuple[float, ...] = (30.0, 60.0, 120.0)
    output_dir: str | None = None
    eval_name: str = "eval"
    run_config: RunConfig = field(default_factory=RunConfig)
    sample_timeout_s: float | None = None        # a sample that runs longer is recorded as failed ("timeout") and the run goes on
    show_progress: bool = False                  # one overall bar plus a line per sample in flight, on stderr


@dataclass
class AgentSession:
    session_id: str
    created_at: float = field(default_factory=time.time)
    updated_at: float = field(default_factory=time.time)
    endpoint: dict[str, Any] = field(default_factory=dict)
    environment: dict[str, Any] | None = None
    parent_id: str | None = None
    branch_point: int | None = None
    status: str = "active"
    tags: dict[str, Any] = field(default_factory=dict)
    num_messages: int = 0


def to_jsonable(obj: Any) -> Any:
    if is_dataclass(obj) and not isinstance(obj, type):
        return {f.name: to_jsonable(getattr(obj, f.name)) for f in fields(obj)}
    if isinstance(obj, Enum):
        return obj.value
    if isinstance(obj, (list, tuple)):
        return [to_jsonable(x) for x in obj]
    if isinstance(obj, dict):
        return {str(k): to_jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (str, int, float, bool)) or obj is None:
        return obj
    return repr(obj)
