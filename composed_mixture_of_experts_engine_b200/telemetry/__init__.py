"""Structured telemetry sinks."""

from .logger import PhaseTimer, PrometheusExporter, StepRecord, StructuredLogger, WandBSink  # noqa: F401

__all__ = ["StepRecord", "StructuredLogger", "WandBSink", "PrometheusExporter", "PhaseTimer"]
