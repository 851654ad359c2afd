"""Root preset for questions that need computation rather than files: a Python scratchpad and web access."""

from ..presets import AgentPresetConfig

config = AgentPresetConfig(name="scratchpad", model="openai/gpt-5.1", env="research", thinking=True, max_turns=30,
                           system_prompt=("Answer with sources. Search and read the pages you cite. Use the Python tool whenever a number matters: "
                                          "compute it, do not estimate it. Show the figures you relied on."),
                           description="web search / fetch plus a persistent Python scratchpad")
