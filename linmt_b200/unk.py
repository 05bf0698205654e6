"""Python mirror of the reference's UNK post-processing class (PostProcessUnks,
src/postprocess_unks.h:25-84) over the C ABI: same method names, same config file."""
from __future__ import annotations

import ctypes as C

from . import _lib


class PostProcessUnks:
    def __init__(self):
        self._lib = _lib.load()
        self._h = C.c_void_p()

    def Init(self, config: str) -> bool:
        self.close()
        rc = self._lib.linmt_unk_create(config.encode(), C.byref(self._h))
        if rc != 0:
            raise RuntimeError(f"linmt_unk_create failed ({rc}): missing config or resource file")
        return True

    def Process(self, source_sentence: str, input_sentence: str) -> str:
        """Returns the whole post-processed line (words and the unchanged `||||` fields)."""
        cap = 4 * (len(source_sentence.encode()) + len(input_sentence.encode())) + 4096
        buf = C.create_string_buffer(cap)
        rc = self._lib.linmt_unk_process(self._h, source_sentence.encode(), input_sentence.encode(), buf, cap)
        if rc != 0:
            raise RuntimeError(f"linmt_unk_process failed ({rc})")
        return buf.value.decode()

    def close(self):
        if self._h:
            self._lib.linmt_unk_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def unk_init(config: str) -> None:
    """python_unk_init (process-wide singleton, exits on a missing file like the reference)."""
    _lib.load().python_unk_init(config.encode())


def unk_do_job(src_sentence: str, translation: str) -> str:
    """python_unk_do_job: the final words only."""
    return _lib.load().python_unk_do_job(src_sentence.encode(), translation.encode()).decode()
