"""distdl_b200: a Blackwell-native partitioned-tensor parallelism framework."""
__version__ = "0.1.0"
