"""B200-native decode-step runtime behind TileFoundry's runtime-twin boundary."""
__version__ = "0.1.0"
