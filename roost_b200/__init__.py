"""roost_b200: a small, whole inference engine for the dense Qwen3 decoder on one B200 (sm_100a).

Public entry points: ``RoostEngine`` (token ids in, generated ids out; with a caller's tokenizer also text and chat
messages in, text out, with stop strings), ``GenerationOptions``,
``SamplingParameters``, ``StepExecutor``/``StepEntry`` (the raw step function), ``load_model``,
``write_random_model``; the command line is ``bin/roost`` and the replay tool ``bin/trace_run``.
"""
from .engine.engine import Completion, CompletionUpdate, GenerationOptions, RoostEngine
from .engine.executor import StepEntry, StepError, StepExecutor
from .engine.model import Model, load_model, read_model_config
from .engine.request import GREEDY, Request, RequestError, SamplingParameters, TokenEvent
from .engine.scheduler import Scheduler, SchedulerOptions
from .engine.text import IncrementalDetokenizer, StopMatcher, TextCompletion, TextUpdate, render_chat
from .registry import register_architecture
from .weights.random_init import write_random_model

__version__ = "0.1.0"
__all__ = ["Completion", "CompletionUpdate", "GenerationOptions", "RoostEngine", "StepEntry", "StepError", "StepExecutor", "Model",
           "load_model", "read_model_config", "GREEDY", "Request", "RequestError", "SamplingParameters", "TokenEvent", "Scheduler",
           "SchedulerOptions", "register_architecture", "write_random_model", "IncrementalDetokenizer", "StopMatcher", "TextCompletion",
           "TextUpdate", "render_chat"]
