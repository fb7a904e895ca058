from .streams import get_stream_context, record_event, synchronize  # noqa: F401
