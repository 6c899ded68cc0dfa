"""Cache directory tree (same folder names as the reference, classes/paths.py:9-37):

    <cache>/dataset/distributions.hdf5
    <cache>/dataset/validation/distributions.hdf5
    <cache>/student/{states,gguf,trained}/
"""
from __future__ import annotations

import os
import shutil
from pathlib import Path


class Paths:
    H5_NAME = "distributions.hdf5"

    def __init__(self, cache: str, clean_start: bool = False):
        self.cache = str(cache)
        self.dataset = os.path.join(self.cache, "dataset")
        self.dataset_validation = os.path.join(self.dataset, "validation")
        self.student_root = os.path.join(self.cache, "student")
        self.student_states = os.path.join(self.student_root, "states")
        self.student_gguf = os.path.join(self.student_root, "gguf")
        self.student_trained = os.path.join(self.student_root, "trained")
        if clean_start:
            self.empty_all()
        for d in (self.cache, self.dataset, self.dataset_validation, self.student_root, self.student_states,
                  self.student_gguf, self.student_trained):
            os.makedirs(d, exist_ok=True)

    # ---- queries (the reference's versions call a non-existent os.join, classes/paths.py:43-47)
    @property
    def h5_main(self) -> str:
        return os.path.join(self.dataset, self.H5_NAME)

    @property
    def h5_validation(self) -> str:
        return os.path.join(self.dataset_validation, self.H5_NAME)

    def dataset_present(self) -> bool:
        return os.path.exists(self.h5_main)

    def validation_present(self) -> bool:
        return os.path.exists(self.h5_validation)

    def create_folder(self, existing_folder: str, subfolder: str) -> str:
        p = os.path.join(existing_folder, subfolder)
        os.makedirs(p, exist_ok=True)
        setattr(self, subfolder, p)
        return p

    # ---- cleanup
    @staticmethod
    def empty_folder(folder: str) -> None:
        root = Path(folder)
        if not root.exists():
            return
        for entry in root.iterdir():
            if entry.is_dir() and not entry.is_symlink():
                shutil.rmtree(entry)
            else:
                entry.unlink()

    def empty_dataset(self) -> None:
        self.empty_folder(self.dataset)

    def empty_student_root(self) -> None:
        self.empty_folder(self.student_root)

    def empty_student_states(self) -> None:
        self.empty_folder(self.student_states)

    def empty_all(self) -> None:
        self.empty_dataset()
        self.empty_student_root()
