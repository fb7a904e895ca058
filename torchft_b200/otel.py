"""Structured event loggers (quorum changes, commit votes, communicator aborts).

Three named loggers carry one record per event with the fields ``job_id, replica_id,
rank, quorum_id, step`` plus ``commit_result`` or ``error`` in ``extra``:
``torchft_quorums``, ``torchft_commits`` and ``torchft_errors``.  :func:`setup_logger`
attaches a console handler that prints those fields and, when the OpenTelemetry SDK is
importable and ``TORCHFT_USE_OTEL`` is not ``false``, an OTLP/HTTP exporter whose
resource attributes come from the JSON file named by
``TORCHFT_OTEL_RESOURCE_ATTRIBUTES_JSON``.  Role of torchft/otel.py:24-84.
"""

from __future__ import annotations

import json
import logging
import os
import time
from typing import Optional

TORCHFT_USE_OTEL = "TORCHFT_USE_OTEL"
TORCHFT_OTEL_RESOURCE_ATTRIBUTES_JSON = "TORCHFT_OTEL_RESOURCE_ATTRIBUTES_JSON"

_FIELDS = ("job_id", "replica_id", "rank", "quorum_id", "step", "commit_result", "error")
_configured: set = set()


class _FieldFormatter(logging.Formatter):
    def format(self, record: logging.LogRecord) -> str:
        parts = [f"{k}={getattr(record, k)}" for k in _FIELDS if hasattr(record, k)]
        msg = record.getMessage()
        ts = time.strftime("%Y-%m-%dT%H:%M:%S", time.localtime(record.created))
        return f"{ts} {record.name} {' '.join(parts)}{(' ' + msg) if msg else ''}"


def _otel_handler(name: str) -> Optional[logging.Handler]:
    if os.environ.get(TORCHFT_USE_OTEL, "false").lower() == "false":
        return None
    try:
        from opentelemetry._logs import set_logger_provider  # noqa: F401
        from opentelemetry.exporter.otlp.proto.http._log_exporter import OTLPLogExporter
        from opentelemetry.sdk._logs import LoggerProvider, LoggingHandler
        from opentelemetry.sdk._logs.export import BatchLogRecordProcessor
        from opentelemetry.sdk.resources import Resource
    except Exception:
        logging.getLogger(__name__).warning("TORCHFT_USE_OTEL is set but the OpenTelemetry SDK is not installed")
        return None
    attrs = {}
    path = os.environ.get(TORCHFT_OTEL_RESOURCE_ATTRIBUTES_JSON)
    if path:
        with open(path) as f:
            attrs = json.load(f).get(name, {})
    provider = LoggerProvider(resource=Resource.create(attrs))
    provider.add_log_record_processor(BatchLogRecordProcessor(OTLPLogExporter(timeout=5)))
    return LoggingHandler(level=logging.NOTSET, logger_provider=provider)


def setup_logger(name: str) -> logging.Logger:
    """Idempotently configure one of the structured loggers."""
    logger = logging.getLogger(name)
    if name in _configured:
        return logger
    _configured.add(name)
    logger.setLevel(logging.INFO)
    logger.propagate = False
    if os.environ.get("TORCHFT_B200_EVENT_CONSOLE", "0") == "1":
        h = logging.StreamHandler()
        h.setFormatter(_FieldFormatter())
        logger.addHandler(h)
    else:
        logger.addHandler(logging.NullHandler())
    oh = _otel_handler(name)
    if oh is not None:
        logger.addHandler(oh)
    return logger
