"""Distributed training: flat buffers, data / ZeRO / tensor / pipeline parallel, collectives over peer memory."""
from .flat import FlatBuffers

__all__ = ["FlatBuffers"]
