"""Single-process tools "corresponding to the parallel version" (reference: tool/README.md:1,
tool/*.cpp, tool/balltree/, tool/datagen.py).  Each module has a ``main(cfg_file)`` that
reads the same JSON keys as the reference executable and writes the same dump files."""
