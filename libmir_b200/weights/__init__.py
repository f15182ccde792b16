from .loader import canonical, catalog_shapes, load_into, match
from .random_init import bind_random, parameter_specs, random_tensor, write_model_folder
from .safetensors_io import TensorEntry, load_tensor, read_catalog, read_header, write_file

__all__ = ["TensorEntry", "bind_random", "canonical", "catalog_shapes", "load_into", "load_tensor", "match",
           "parameter_specs", "random_tensor", "read_catalog", "read_header", "write_file", "write_model_folder"]
