"""Flat index of a Cartesian index in row-major (C) or column-major (F) order."""


def cartesian_index_c(shape, index):
    flat = 0
    for n, i in zip(shape, index):
        flat = flat * int(n) + int(i)
    return flat


def cartesian_index_f(shape, index):
    flat = 0
    for n, i in zip(reversed(list(shape)), reversed(list(index))):
        flat = flat * int(n) + int(i)
    return flat
