from .arena import ArenaPlan, FileSource, FusedSpec, MappedFile, Piece, RandomSource, WeightArena
from .loader import WeightError, WeightSpec, load_weights, plan_arena, read_weights, storage_dtype
from .random_init import draw_cpu, random_weights_cpu, write_random_model
from .safetensors_io import SafetensorsError, SafetensorsFile, save_safetensors

__all__ = ["ArenaPlan", "FileSource", "FusedSpec", "MappedFile", "Piece", "RandomSource", "WeightArena",
           "WeightError", "WeightSpec", "load_weights", "plan_arena", "read_weights", "storage_dtype", "draw_cpu",
           "random_weights_cpu", "write_random_model", "SafetensorsError", "SafetensorsFile", "save_safetensors"]
