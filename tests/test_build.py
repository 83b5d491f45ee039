"""Where compiled kernels are kept and which folders' libraries are trusted (no GPU, no compiler)."""
from __future__ import annotations

import os
import tempfile
from pathlib import Path

from thintensor_b200.kernels import build


def test_a_folder_others_can_write_to_is_not_trusted(tmp_path):
    mine = tmp_path / "mine"
    mine.mkdir(mode=0o700)
    assert build._is_private(mine)
    shared = tmp_path / "shared"
    shared.mkdir()
    os.chmod(shared, 0o777)
    assert not build._is_private(shared)
    group = tmp_path / "group"
    group.mkdir()
    os.chmod(group, 0o770)
    assert not build._is_private(group)
    link = tmp_path / "link"
    link.symlink_to(mine, target_is_directory=True)
    assert not build._is_private(link), "a symbolic link may point anywhere"
    assert not build._is_private(tmp_path / "absent")


def test_the_temporary_build_folder_is_private_even_if_its_name_is_taken(tmp_path, monkeypatch):
    monkeypatch.setattr(tempfile, "tempdir", str(tmp_path))
    first = build._private_temp_folder()
    assert first == tmp_path / f"thintensor_b200-build-{os.getuid()}" and build._is_private(first)
    assert build._private_temp_folder() == first                    # found again, still private
    os.chmod(first, 0o777)                                          # as if somebody else had made it
    other = build._private_temp_folder()
    assert other != first and build._is_private(other) and Path(other).parent == tmp_path


def test_libraries_are_looked_for_in_trusted_folders_only(tmp_path, monkeypatch):
    """A library of the right name in the shared temporary directory's per-user folder is not
    picked up unless that folder is the checked build folder of this process."""
    monkeypatch.setattr(tempfile, "tempdir", str(tmp_path))
    planted = tmp_path / f"thintensor_b200-build-{os.getuid()}"
    planted.mkdir()
    os.chmod(planted, 0o777)
    name = "elementwise"
    (planted / build.library_path(name, planted).name).write_bytes(b"not a library")
    chosen = tmp_path / "chosen"
    chosen.mkdir(mode=0o700)
    monkeypatch.setattr(build, "_build_dir", chosen)
    found = build._find_built(name)
    assert found is None or found.parent != planted
