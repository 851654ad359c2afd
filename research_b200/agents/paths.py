"""Where this package, its documentation and its presets live on disk (rollouts/paths.py:21-101), so that an agent
asked about its own capabilities can be pointed at files that exist."""

from __future__ import annotations

from pathlib import Path


def get_version() -> str:
    """The installed distribution's version, else the one in ``pyproject.toml`` beside the package, else ``"dev"``."""
    try:
        from importlib.metadata import PackageNotFoundError, version

        try:
            return version("research_b200")
        except PackageNotFoundError:
            pass
    except ImportError:  # pragma: no cover
        pass
    pyproject = get_repo_root() / "pyproject.toml"
    if pyproject.is_file():
        for line in pyproject.read_text().splitlines():
            if line.strip().startswith("version") and "=" in line:
                return line.split("=", 1)[1].strip().strip("\"'")
    return "dev"


def get_package_dir() -> Path:
    return Path(__file__).resolve().parent.parent


def get_repo_root() -> Path:
    return get_package_dir().parent


def get_readme_path() -> Path:
    return get_repo_root() / "README.md"


def get_docs_dir() -> Path:
    """The folder with the longer documents (the repository root: design notes and profiles live beside the README)."""
    return get_repo_root()


def get_presets_dir() -> Path:
    return get_package_dir() / "agents"


def get_readme_content() -> str | None:
    p = get_readme_path()
    return p.read_text() if p.is_file() else None


def get_doc_content(name: str) -> str | None:
    """A document of the documentation folder by file name (``None`` if there is none; no path components allowed)."""
    if "/" in name or "\\" in name or name.startswith("."):
        return None
    p = get_docs_dir() / name
    return p.read_text() if p.is_file() else None
