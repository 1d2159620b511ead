"""Diagnostics: telemetry bus and hooks, profiler, kernel timing, setting advisor."""
from .telemetry import (BatchCompleted, ChannelTelemetry, ConsoleLogger, EpochCompleted, Event, JsonLinesLogger, Level,
                        MetricsRecorder, Telemetry, TelemetryHook)

__all__ = ["BatchCompleted", "ChannelTelemetry", "ConsoleLogger", "EpochCompleted", "Event", "JsonLinesLogger", "Level",
           "MetricsRecorder", "Telemetry", "TelemetryHook"]
