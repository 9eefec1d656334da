"""paracel_b200: a Blackwell-native parameter-server ML framework with the
programming model, algorithm suite and dump formats of douban/paracel."""
__version__ = "0.1.0"
