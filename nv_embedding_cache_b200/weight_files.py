"""Weight files either side of the lookup path: the ``.nve`` tensor container and the two table
file formats the reference loads tables from (``include/serialization.hpp:54-141``,
``src/serialization.cpp``).  Byte-compatible with the reference in both directions.

``.nve`` container (little endian):

    header   uint32 magic 0x4e564500, uint32 version major 0, uint32 version minor 2
    entries  one after another, each
               uint64 key1   = cols | elem_bytes << 16 | rows << 20
               uint64 key2   = tensor name (an integer id)
               uint64 offset = file position of the next entry
               uint64 length = rows * cols * elem_bytes
               length bytes of row-major data

Table files: a raw binary file of fixed-size rows (``BinaryTable``), or a ``.npy`` file, format
version 1.0 or 2.0, dtype <f4 / <f8 / <i4 / <i8, C order (``NumpyTable``); both hand out rows in
batches, the way a layer is filled from them.
"""
from __future__ import annotations

import io
import re
import struct
from typing import BinaryIO

import numpy as np

MAGIC_NUMBER = 0x4E564500
VERSION_MAJOR, VERSION_MINOR = 0, 2
_HEADER = struct.Struct("<III")
_ENTRY = struct.Struct("<QQQQ")
_ROW_SIZE_BITS, _DATA_TYPE_BITS = 16, 4
_ROWS_BITS = 64 - _ROW_SIZE_BITS - _DATA_TYPE_BITS


def _tensor_key(rows: int, cols: int, elem_bytes: int) -> int:
    if cols >= 1 << _ROW_SIZE_BITS:
        raise ValueError("nve support max 16 bit row size")
    if rows >= 1 << _ROWS_BITS:
        raise ValueError("nve support max 44 bit rows")
    if elem_bytes >= 1 << _DATA_TYPE_BITS:
        raise ValueError("nve support max 2 bit data type")
    return cols | elem_bytes << _ROW_SIZE_BITS | rows << (_ROW_SIZE_BITS + _DATA_TYPE_BITS)


def write_header(stream: BinaryIO) -> None:
    """reference TensorFileFormat::write_table_file_header"""
    stream.seek(0)
    stream.write(_HEADER.pack(MAGIC_NUMBER, VERSION_MAJOR, VERSION_MINOR))
    stream.flush()


def verify_header(stream: BinaryIO) -> bool:
    stream.seek(0)
    raw = stream.read(_HEADER.size)
    return len(raw) == _HEADER.size and _HEADER.unpack(raw) == (MAGIC_NUMBER, VERSION_MAJOR, VERSION_MINOR)


def write_tensor(stream: BinaryIO, name: int, tensor) -> None:
    """Appends a 2-D tensor at the stream's position (reference write_tensor_to_stream)."""
    a = np.ascontiguousarray(tensor)
    if a.ndim != 2:
        raise ValueError("a table is a 2-D tensor")
    size = a.shape[0] * a.shape[1] * a.itemsize
    key1 = _tensor_key(a.shape[0], a.shape[1], a.itemsize)
    stream.write(_ENTRY.pack(key1, name, size + _ENTRY.size + stream.tell(), size))
    stream.write(a.tobytes())
    stream.flush()


def read_tensor(stream: BinaryIO, name: int, out: np.ndarray) -> bool:
    """Fills ``out`` (2-D, C-contiguous) with tensor ``name``; False when the file holds no such
    tensor (the reference leaves the destination untouched in that case).  The stored byte length
    must equal that of ``out`` (reference load_tensor_from_stream)."""
    if not verify_header(stream):
        raise ValueError("Incorrect file version")
    if out.ndim != 2 or not out.flags.c_contiguous:
        raise ValueError("destination must be a C-contiguous 2-D array")
    while True:
        raw = stream.read(_ENTRY.size)
        if len(raw) == 0:
            return False
        if len(raw) != _ENTRY.size:
            raise ValueError("Problem reading table entry")
        _, key2, offset, length = _ENTRY.unpack(raw)
        if key2 == name:
            if length != out.nbytes:
                raise ValueError("Incorrect tensor size")
            data = stream.read(length)
            if len(data) != length:
                raise ValueError("Problem reading tensor")
            out.view(np.uint8).reshape(-1)[:] = np.frombuffer(data, np.uint8)
            return True
        stream.seek(offset)


def list_tensors(stream: BinaryIO):
    """(name, rows, cols, elem_bytes) of every tensor in a .nve stream, in file order."""
    if not verify_header(stream):
        raise ValueError("Incorrect file version")
    found = []
    while True:
        raw = stream.read(_ENTRY.size)
        if len(raw) == 0:
            return found
        if len(raw) != _ENTRY.size:
            raise ValueError("Problem reading table entry")
        key1, key2, offset, _ = _ENTRY.unpack(raw)
        found.append((key2, key1 >> (_ROW_SIZE_BITS + _DATA_TYPE_BITS), key1 & ((1 << _ROW_SIZE_BITS) - 1),
                      (key1 >> _ROW_SIZE_BITS) & ((1 << _DATA_TYPE_BITS) - 1)))
        stream.seek(offset)


class BinaryTable:
    """Raw binary table file: ``row_size_in_bytes`` per row, as many whole rows as the file holds
    (reference BinaryTensorFileFormat)."""

    def __init__(self, stream: BinaryIO, row_size_in_bytes: int):
        if row_size_in_bytes <= 0:
            raise ValueError("row size must be positive")
        self._stream = stream
        self._row = row_size_in_bytes

    def get_num_rows(self) -> int:
        at = self._stream.tell()
        end = self._stream.seek(0, io.SEEK_END)
        self._stream.seek(at)
        return end // self._row

    def get_row_size_in_bytes(self) -> int:
        return self._row

    def reset(self) -> None:
        self._stream.seek(0)

    def load_batch(self, batch: int) -> np.ndarray:
        """The next ``batch`` rows as a [batch, row bytes] uint8 array."""
        want = batch * self._row
        data = self._stream.read(want)
        if len(data) != want:
            raise ValueError("table file ends inside the requested batch")
        return np.frombuffer(data, np.uint8).reshape(batch, self._row)


_NPY_MAGIC = b"\x93NUMPY"
_NPY_ITEMSIZE = {"<f4": 4, "<f8": 8, "<i4": 4, "<i8": 8}


class NumpyTable:
    """``.npy`` table file read as rows of ``prod(shape[1:])`` elements (reference
    NumpyTensorFileFormat): versions 1.0 and 2.0, dtypes <f4 <f8 <i4 <i8, and a file that is too
    short for its declared shape is refused when it is opened."""

    def __init__(self, stream: BinaryIO):
        self._stream = stream
        stream.seek(0)
        if stream.read(len(_NPY_MAGIC)) != _NPY_MAGIC:
            raise ValueError("Incorrect file format")
        version = stream.read(2)
        if len(version) != 2:
            raise ValueError("Problem reading numpy version")
        if tuple(version) == (1, 0):
            len_bytes = 2
        elif tuple(version) == (2, 0):
            len_bytes = 4
        else:
            raise ValueError("Unsupported numpy version")
        raw = stream.read(len_bytes)
        if len(raw) != len_bytes:
            raise ValueError("Problem reading numpy header length")
        header_len = int.from_bytes(raw, "little")
        header = stream.read(header_len)
        if len(header) != header_len:
            raise ValueError("Problem reading numpy header")
        text = header.decode("latin1")
        m = re.search(r"'descr': '([^']+)'", text)
        if not m:
            raise ValueError("Incorrect file format")
        if m.group(1) not in _NPY_ITEMSIZE:
            raise ValueError("Unsupported data type")
        self.descr = m.group(1)
        self._itemsize = _NPY_ITEMSIZE[self.descr]
        m = re.search(r"shape': \(([^)]*)\)", text)
        if not m:
            raise ValueError("Incorrect file format")
        shape = []
        for token in m.group(1).split(","):
            token = token.strip(" \t")
            if token == "":
                continue                      # after the trailing comma of "(5,)"
            if not token.isdigit() or not token.isascii():
                raise ValueError(f"Failed to parse numpy shape: '{m.group(1)}'")
            shape.append(int(token))
        if not shape:
            raise ValueError("Empty numpy shape")
        self._shape = shape
        m = re.search(r"fortran_order': (False|True)", text)
        if not m:
            raise ValueError("Incorrect file format")
        self.fortran_order = m.group(1) == "True"
        self._offset = stream.tell()
        vec = 1
        for d in shape[1:]:
            vec *= d
        self._row = vec * self._itemsize
        if self._row >= 1 << 64 or shape[0] * self._row >= 1 << 64:
            raise ValueError("Numpy data size computation overflows uint64")
        end = stream.seek(0, io.SEEK_END)
        stream.seek(self._offset)
        if end - self._offset < shape[0] * self._row:
            raise ValueError(f"Numpy file too small for declared shape: needs {shape[0] * self._row} "
                             f"bytes after header, has {end - self._offset}")

    def get_num_rows(self) -> int:
        return self._shape[0]

    def get_shape(self):
        return list(self._shape)

    def get_row_size_in_bytes(self) -> int:
        return self._row

    def reset(self) -> None:
        self._stream.seek(self._offset)

    def load_batch(self, batch: int) -> np.ndarray:
        want = batch * self._row
        data = self._stream.read(want)
        if len(data) != want:
            raise ValueError("table file ends inside the requested batch")
        return np.frombuffer(data, np.uint8).reshape(batch, self._row)


def load_table(table_file, destination: np.ndarray, batch_rows: int = 1 << 16) -> int:
    """Streams every row of a BinaryTable / NumpyTable into ``destination`` (a [rows, row bytes]
    uint8 view of the table storage) in batches; returns the number of rows loaded."""
    rows = table_file.get_num_rows()
    if destination.shape[0] < rows or destination.shape[1] != table_file.get_row_size_in_bytes():
        raise ValueError("destination does not fit the table file")
    table_file.reset()
    for r0 in range(0, rows, batch_rows):
        n = min(batch_rows, rows - r0)
        destination[r0:r0 + n] = table_file.load_batch(n)
    return rows
