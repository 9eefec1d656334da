"""Example user handler file: the Python counterpart of the shared objects the reference
loads with dlopen (src/local.cpp:19-46, external_usage/registery.cpp)."""


def multiply(old, delta):
    return old * delta


def starts_with_k(key):
    return key.startswith("k")


def big_values(key, value):
    return isinstance(value, (int, float)) and value > 2
