from .decoder import DecoderModel, Run

__all__ = ["DecoderModel", "Run"]
