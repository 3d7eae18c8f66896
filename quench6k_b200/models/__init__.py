from .decoder import DecoderModel   # noqa: F401
