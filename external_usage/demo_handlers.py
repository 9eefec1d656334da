"""Handler file of the demo application: functions are looked up by name on the servers."""


def add_counts(old, delta):
    return old + delta


def length_keys(key):
    return key.startswith("len_")
