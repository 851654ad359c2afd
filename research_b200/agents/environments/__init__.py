from .basic import BasicEnvironment, BinarySearchEnvironment, CalculatorEnvironment, ComposedEnvironment, compose, safe_eval
from .chess_puzzle import Board, ChessPuzzleEnvironment
from .coding import LocalFilesystemEnvironment, MessageParsingREPLEnvironment, REPLEnvironment
from .git_worktree import GitWorktreeEnvironment
from .interactive import AskUserQuestionEnvironment, BrowsingEnvironment, ScreenSpotEnvironment
from .rlm import MessageParsingRLMEnvironment, RLMEnvironment

__all__ = ["BasicEnvironment", "BinarySearchEnvironment", "CalculatorEnvironment", "ComposedEnvironment", "compose", "safe_eval",
           "LocalFilesystemEnvironment", "MessageParsingREPLEnvironment", "REPLEnvironment", "Board",
           "ChessPuzzleEnvironment", "GitWorktreeEnvironment", "AskUserQuestionEnvironment", "BrowsingEnvironment",
           "ScreenSpotEnvironment", "RLMEnvironment", "MessageParsingRLMEnvironment"]
