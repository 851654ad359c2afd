"""Agent runtime: data types, the agent loop, providers, environments, evaluation, sessions, search."""

from .agents import (compose_stop_handlers, handle_no_tool_continue, handle_no_tool_stop, handle_stop_max_turns,
                     process_pending_tools, resume_session, rollout, run_agent, run_agent_step)
from .dtypes import (Actor, AgentSession, AgentState, ChatCompletion, Choice, Cost, Endpoint, Environment, EvalConfig,
                     Logprob, Logprobs, Message, Metric, RunConfig, Score, StopReason, TextContent, ThinkingContent, Tool,
                     ToolCall, ToolCallContent, ToolFunction, ToolFunctionParameter, ToolResult, Trajectory, Usage)
from .evaluation import EvalReport, EvalSample, compute_summary_metrics, evaluate, evaluate_sample, group_by, summarize
from .search import SearchNode, prune, run_search, select_best
from .store import FileSessionStore, SessionStore, log_crash

__all__ = [n for n in dir() if not n.startswith("_")]
