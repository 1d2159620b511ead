"""Serving: paged KV cache, continuous-batching engine, multi-model inference engine, HTTP API."""
from .engine import GenerationOptions, LLMEngine, Request, StepOutput
from .runner import ModelRunner, PrefillItem
from .scheduler import QueueFull, Scheduler

__all__ = ["GenerationOptions", "LLMEngine", "Request", "StepOutput", "ModelRunner", "PrefillItem", "QueueFull",
           "Scheduler"]
