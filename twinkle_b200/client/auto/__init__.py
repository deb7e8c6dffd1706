"""``twinkle-auto``: a conversational agent that writes, launches, watches and repairs training scripts.

Parity: reference ``src/twinkle_client/auto/`` (connection, runtime, agent core / tools / monitor / prompts, app) and
``src/twinkle_client/skills/``.

================  ====================================================================================================
``runs``          run directories (script + archived versions, metadata, metrics, combined output) and process control
``runtime``       what a generated script imports: metrics, resume information, save-on-SIGTERM
``llm``           OpenAI-compatible chat client with tool calls (plain and streamed) and a scripted stand-in
``tools``         tool schemas and their executor (runs, local server, cached hub search, host information)
``agent``         the conversation loop with tool rounds, skills in the system prompt, history pruning
``monitor``       periodic health check → LGTM / warning / automatic fix-and-relaunch (at most three per run)
``app``           terminal front end and the ``twinkle-auto`` entry point
================  ====================================================================================================
"""
from .agent import SYSTEM_PROMPT, AgentLoop
from .llm import ChatLLM, ScriptedLLM, merge_stream
from .monitor import MAX_FIX_ATTEMPTS, TrainingMonitor, local_findings, parse_verdict
from .runs import RunStore, pid_state
from .runtime import TrainingRuntime
from .tools import TOOL_SCHEMAS, ToolExecutor, server_config, split_gpus

__all__ = ['AgentLoop', 'SYSTEM_PROMPT', 'ChatLLM', 'ScriptedLLM', 'merge_stream', 'TrainingMonitor', 'MAX_FIX_ATTEMPTS', 'local_findings',
           'parse_verdict', 'RunStore', 'pid_state', 'TrainingRuntime', 'TOOL_SCHEMAS', 'ToolExecutor', 'server_config', 'split_gpus']
