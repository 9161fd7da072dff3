"""HuggingFace Hub client: file lists, metadata, resumable verified downloads.

Protocol facts kept from the reference (``src/exo/download/download_utils.py:64-105, 382-757``,
``huggingface_utils.py:13-171``): endpoint from ``HF_ENDPOINT``; token from ``HF_TOKEN`` or
``$HF_HOME/token``; tree listing at ``/api/models/<id>/tree/<rev>?recursive=true`` cached on disk
(TTL) and falling back to the cache or the local directory when the hub is unreachable; HEAD on
``/<id>/resolve/<rev>/<path>`` gives size and hash (``x-linked-size`` / ``x-linked-etag`` on a 307
are authoritative); bytes stream into ``<file>.partial`` with a ``Range`` request to resume; the
finished file is verified (git-blob SHA-1 for small files, SHA-256 for LFS) before the rename;
401/403 raise at once, 429 honours ``Retry-After``, everything else backs off exponentially for
five attempts.
"""
from __future__ import annotations

import asyncio
import fnmatch
import hashlib
import os
import random
import time
from collections.abc import Callable, Iterable, Mapping
from pathlib import Path
from typing import TypeVar
from urllib.parse import urljoin

import aiohttp
from pydantic import TypeAdapter

from ..shared.base import ModelId
from .store import FileListEntry, cache_dir, scan_model_directory, build_model_path

FILE_LIST_CACHE_TTL_S = 300.0
RATE_LIMIT_MAX_SLEEP_S = 60.0
N_ATTEMPTS = 5
BACKOFF_SCALE_S = 1.0          # tests shrink this
CHUNK = 8 << 20
T = TypeVar("T")
_FileList = TypeAdapter(list[FileListEntry])


class HuggingFaceAuthenticationError(Exception):
    pass


class HuggingFaceRateLimitError(Exception):
    def __init__(self, msg: str, retry_after: float | None = None):
        super().__init__(msg)
        self.retry_after = retry_after


def hf_endpoint() -> str:
    return os.environ.get("HF_ENDPOINT", "https://huggingface.co").rstrip("/")


def hf_home() -> Path:
    return Path(os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface"))


def hf_token() -> str | None:
    tok = os.environ.get("HF_TOKEN")
    if tok:
        return tok.strip()
    p = hf_home() / "token"
    try:
        return p.read_text().strip() or None
    except OSError:
        return None


def auth_headers() -> dict[str, str]:
    tok = hf_token()
    return {"Authorization": f"Bearer {tok}"} if tok else {}


def download_headers() -> dict[str, str]:
    return {**auth_headers(), "Accept-Encoding": "identity"}


def parse_retry_after(headers: Mapping[str, str]) -> float | None:
    v = headers.get("Retry-After") or headers.get("retry-after")
    if v is None:
        # hub rate-limit header: `"api";r=0;t=42` -> seconds until the window resets
        rl = headers.get("RateLimit") or headers.get("ratelimit")
        if rl:
            for part in rl.split(";"):
                part = part.strip()
                if part.startswith("t="):
                    try:
                        return float(part[2:])
                    except ValueError:
                        return None
        return None
    try:
        return max(0.0, float(v))
    except ValueError:
        try:
            from email.utils import parsedate_to_datetime
            return max(0.0, parsedate_to_datetime(v).timestamp() - time.time())
        except (TypeError, ValueError):
            return None


def auth_error_message(status: int, model_id: str) -> str:
    if status == 401 and hf_token() is None:
        return (f"Model '{model_id}' requires authentication. Set HF_TOKEN in the environment, or run "
                f"`hf auth login`, then accept the model's licence at {hf_endpoint()}/{model_id}")
    if status == 403:
        return f"Access denied to '{model_id}'. Accept the model's licence at {hf_endpoint()}/{model_id}"
    return f"Authentication failed for '{model_id}' (HTTP {status}); check that HF_TOKEN is valid"


def trim_etag(etag: str) -> str:
    if etag.startswith("W/"):
        etag = etag[2:]
    etag = etag.strip('"')
    return etag[:-5] if etag.endswith("-gzip") else etag


def filter_repo_objects(items: Iterable[T], *, allow_patterns: list[str] | None = None,
                        ignore_patterns: list[str] | None = None, key: Callable[[T], str] = str) -> Iterable[T]:
    def widen(p: str) -> str:
        return p + "*" if p.endswith("/") else p
    allow = [widen(p) for p in allow_patterns] if allow_patterns is not None else None
    ignore = [widen(p) for p in ignore_patterns] if ignore_patterns is not None else None
    for it in items:
        path = key(it)
        if allow is not None and not any(fnmatch.fnmatch(path, p) for p in allow):
            continue
        if ignore is not None and any(fnmatch.fnmatch(path, p) for p in ignore):
            continue
        yield it


def extract_layer_num(tensor_name: str) -> int | None:
    for part in tensor_name.split("."):
        if part.isdigit():
            return int(part)
    return None


DEFAULT_PATTERNS = ("*.json", "*.py", "tokenizer.model", "tiktoken.model", "*/spiece.model", "*.tiktoken", "*.txt", "*.jinja")


def allow_patterns_for_layers(weight_map: Mapping[str, str], start_layer: int, end_layer: int) -> list[str]:
    """Files a pipeline stage needs: its layers' weight files plus everything that is not per-layer."""
    if not weight_map:
        return [*DEFAULT_PATTERNS, "*.safetensors"]
    files = set()
    for name, fn in weight_map.items():
        n = extract_layer_num(name)
        if n is None or start_layer <= n < end_layer:
            files.add(fn)
    return [*DEFAULT_PATTERNS, *sorted(files)]


def session(profile: str = "long") -> aiohttp.ClientSession:
    to = (aiohttp.ClientTimeout(total=30, connect=10, sock_read=30) if profile == "short"
          else aiohttp.ClientTimeout(total=None, connect=30, sock_read=120))
    return aiohttp.ClientSession(timeout=to, trust_env=True, auto_decompress=False)


async def _raise_for(status: int, headers: Mapping[str, str], model_id: str, what: str) -> None:
    if status in (401, 403):
        raise HuggingFaceAuthenticationError(auth_error_message(status, model_id))
    if status == 429:
        raise HuggingFaceRateLimitError(f"HuggingFace rate limit hit {what} for {model_id}", parse_retry_after(headers))


async def _retrying(fn: Callable[[], "asyncio.Future[T]"], what: str, on_connection_lost: Callable[[], None],
                    passthrough: tuple[type[BaseException], ...] = ()) -> T:
    for attempt in range(N_ATTEMPTS):
        try:
            return await fn()
        except (HuggingFaceAuthenticationError, *passthrough):
            raise
        except HuggingFaceRateLimitError as e:
            if attempt == N_ATTEMPTS - 1:
                raise
            pause = e.retry_after if e.retry_after is not None else 2.0 ** attempt
            await asyncio.sleep(min(pause, RATE_LIMIT_MAX_SLEEP_S) + BACKOFF_SCALE_S * random.uniform(0, 1))
        except Exception:
            on_connection_lost()
            if attempt == N_ATTEMPTS - 1:
                raise
            await asyncio.sleep(BACKOFF_SCALE_S * (2.0 ** attempt + random.uniform(0, 1)))
    raise RuntimeError(f"unreachable: {what}")


async def fetch_file_list(model_id: str, revision: str = "main", recursive: bool = True) -> list[FileListEntry]:
    url = f"{hf_endpoint()}/api/models/{model_id}/tree/{revision}" + ("?recursive=true" if recursive else "")
    async with session("short") as s, s.get(url, headers=download_headers()) as r:
        await _raise_for(r.status, r.headers, model_id, "fetching file list")
        if r.status != 200:
            raise RuntimeError(f"Failed to fetch file list: {r.status}")
        return [e for e in _FileList.validate_json(await r.read()) if e.type == "file"]


async def fetch_file_list_with_cache(model_id: ModelId, revision: str = "main", *, skip_internet: bool = False,
                                     on_connection_lost: Callable[[], None] = lambda: None) -> list[FileListEntry]:
    cache_file = cache_dir(model_id) / f"{ModelId(model_id).normalize()}--{revision}--file_list.json"

    def cached() -> list[FileListEntry] | None:
        try:
            return _FileList.validate_json(cache_file.read_bytes())
        except (OSError, ValueError):
            return None

    def local() -> list[FileListEntry] | None:
        d = build_model_path(model_id)
        return scan_model_directory(d) if d.is_dir() else None

    if cache_file.exists() and time.time() - cache_file.stat().st_mtime < FILE_LIST_CACHE_TTL_S:
        if (c := cached()) is not None:
            return c
    if skip_internet:
        got = cached() or local()
        if got is None:
            raise FileNotFoundError(f"No internet connection and no cached file list for {model_id}")
        return got
    try:
        files = await _retrying(lambda: fetch_file_list(str(model_id), revision), "file list", on_connection_lost)
        cache_file.write_bytes(_FileList.dump_json(files))
        return files
    except HuggingFaceAuthenticationError:
        raise
    except Exception as e:
        got = cached() or local()
        if got is None:
            raise FileNotFoundError(f"Failed to fetch file list for {model_id}: {e}") from e
        return got


async def file_meta(model_id: str, revision: str, path: str, redirected: str | None = None, depth: int = 0) -> tuple[int, str]:
    url = (urljoin(f"{hf_endpoint()}/{model_id}/resolve/{revision}/", path) if redirected is None
           else (redirected if redirected.startswith("http") else f"{hf_endpoint()}{redirected}"))
    async with session("short") as s, s.head(url, headers=download_headers(), allow_redirects=False) as r:
        if r.status in (301, 302, 307, 308):
            size, etag = r.headers.get("x-linked-size"), r.headers.get("x-linked-etag")
            if size and etag:
                return int(size), trim_etag(etag)
            loc = r.headers.get("location")
            if loc is None or depth > 4:
                raise RuntimeError(f"redirect without location for {url}")
            return await file_meta(model_id, revision, path, loc, depth + 1)
        await _raise_for(r.status, r.headers, model_id, f"fetching metadata of {path}")
        if r.status == 404:
            raise FileNotFoundError(f"File not found: {url}")
        size = int(r.headers.get("x-linked-size") or r.headers.get("content-length") or 0)
        etag = r.headers.get("x-linked-etag") or r.headers.get("etag")
        if size <= 0 or etag is None:
            raise RuntimeError(f"No size or hash for {url}")
        return size, trim_etag(etag)


def calc_hash(path: Path, kind: str) -> str:
    h = hashlib.sha1() if kind == "sha1" else hashlib.sha256()
    if kind == "sha1":   # git blob id
        h.update(f"blob {path.stat().st_size}\0".encode())
    with open(path, "rb") as f:
        while chunk := f.read(CHUNK):
            h.update(chunk)
    return h.hexdigest()


async def _download_file(model_id: str, revision: str, path: str, target_dir: Path,
                         on_progress: Callable[[int, int, bool], None], skip_internet: bool) -> Path:
    target = target_dir / path
    if target.exists():
        if skip_internet:
            return target
        try:
            remote_size, _ = await file_meta(model_id, revision, path)
        except Exception:
            return target      # offline: trust the local file
        if target.stat().st_size == remote_size:
            return target
        target.unlink()
    if skip_internet:
        raise FileNotFoundError(f"File {path} not found locally and cannot download in offline mode")
    target.parent.mkdir(parents=True, exist_ok=True)
    length, remote_hash = await file_meta(model_id, revision, path)
    partial = target_dir / f"{path}.partial"
    have = partial.stat().st_size if partial.exists() else 0
    if have > length:
        partial.unlink()
        have = 0
    if have != length:
        headers = download_headers()
        if have:
            headers["Range"] = f"bytes={have}-"
        url = urljoin(f"{hf_endpoint()}/{model_id}/resolve/{revision}/", path)
        async with session("long") as s, s.get(url, headers=headers) as r:
            if r.status == 404:
                raise FileNotFoundError(f"File not found: {url}")
            await _raise_for(r.status, r.headers, model_id, f"downloading {path}")
            if r.status not in (200, 206):
                raise RuntimeError(f"Failed to download {path} from {url}: {r.status}")
            if have and r.status == 200:     # server ignored the range: start over
                have = 0
            n = have
            with open(partial, "ab" if have else "wb") as f:
                while chunk := await r.content.read(CHUNK):
                    await asyncio.to_thread(f.write, chunk)
                    n += len(chunk)
                    on_progress(n, length, False)
    digest = await asyncio.to_thread(calc_hash, partial, "sha256" if len(remote_hash) == 64 else "sha1")
    if digest != remote_hash:
        partial.unlink(missing_ok=True)
        raise RuntimeError(f"Downloaded file {target} has hash {digest} but remote hash is {remote_hash}")
    os.replace(partial, target)
    on_progress(length, length, True)
    return target


async def download_file_with_retry(model_id: str, revision: str, path: str, target_dir: Path,
                                   on_progress: Callable[[int, int, bool], None] = lambda a, b, c: None,
                                   on_connection_lost: Callable[[], None] = lambda: None, skip_internet: bool = False) -> Path:
    return await _retrying(lambda: _download_file(model_id, revision, path, target_dir, on_progress, skip_internet),
                           f"download {path}", on_connection_lost, passthrough=(FileNotFoundError,))
