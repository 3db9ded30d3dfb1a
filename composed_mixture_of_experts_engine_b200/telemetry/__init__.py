"""Structured telemetry sinks."""

from .logger import (DeviceClockReader, PhaseTimer, PrometheusExporter, StepRecord, StructuredLogger,  # noqa: F401
                     WandBSink)

__all__ = ["StepRecord", "StructuredLogger", "WandBSink", "PrometheusExporter", "PhaseTimer"]
