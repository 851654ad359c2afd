from .basic import BasicEnvironment, BinarySearchEnvironment, CalculatorEnvironment, ComposedEnvironment, safe_eval
from .coding import LocalFilesystemEnvironment, MessageParsingREPLEnvironment, REPLEnvironment

__all__ = ["BasicEnvironment", "BinarySearchEnvironment", "CalculatorEnvironment", "ComposedEnvironment", "safe_eval",
           "LocalFilesystemEnvironment", "MessageParsingREPLEnvironment", "REPLEnvironment"]
