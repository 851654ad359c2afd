"""Derived from careful_coder_01_01 (parent 01, self 02): a small fast model without extended thinking, for quick
edits and questions about the code; the working rules stay."""

from dataclasses import replace

from .careful_coder_01_01 import config as parent_config

config = replace(parent_config, name="fast_coder", model="anthropic/claude-haiku-4-5", thinking=False, max_turns=30,
                 system_prompt=parent_config.system_prompt + "\n\nPrefer short answers. If the task is larger than a few edits, say so and outline a plan instead.",
                 description="quick edits and code questions with a small model")
