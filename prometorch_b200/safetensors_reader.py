"""Name kept from the reference's package (python/promethorch/safetensors_reader.py): the reader lives in
:mod:`prometorch_b200.io.safetensors`."""
from .io.safetensors import SafeTensorsFile, load_file, load_index, save_file  # noqa: F401

__all__ = ["SafeTensorsFile", "load_file", "load_index", "save_file"]
