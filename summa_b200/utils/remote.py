"""Remote artifact cache: `http(s)://`, `s3://`, `gs://` URIs are fetched once into
`$SUMMA_CACHE` (default `~/.summa-cache`) with 16 MiB ranged GETs, written to a `.part`
file and renamed into place; credentials never appear in messages
(`summa-llm/src/remote.rs:41-168`). Plain paths pass through unchanged."""
from __future__ import annotations

import hashlib
import os
import re
import urllib.request

CHUNK = 16 * 1024 * 1024


def redact(uri: str) -> str:
    uri = re.sub(r"//[^/@]*@", "//***@", uri)
    return re.sub(r"([?&](?:X-Amz-[^=]*|Signature|token|sig|key)=)[^&]*", r"\1***", uri, flags=re.I)


def cache_dir() -> str:
    return os.environ.get("SUMMA_CACHE") or os.path.join(os.path.expanduser("~"), ".summa-cache")


def _http_url(uri: str) -> str:
    if uri.startswith("s3://"):
        bucket, _, key = uri[5:].partition("/")
        return f"https://{bucket}.s3.amazonaws.com/{key}"
    if uri.startswith("gs://"):
        bucket, _, key = uri[5:].partition("/")
        return f"https://storage.googleapis.com/{bucket}/{key}"
    return uri


def resolve(uri: str, opener=None) -> str:
    """Local path for `uri`, downloading it into the cache when it is remote."""
    if not re.match(r"^(https?|s3|gs)://", uri or ""):
        return uri
    name = hashlib.sha256(uri.encode()).hexdigest()[:32] + "-" + os.path.basename(uri.split("?")[0])
    dst = os.path.join(cache_dir(), name)
    if os.path.exists(dst):
        return dst
    os.makedirs(cache_dir(), exist_ok=True)
    part = dst + ".part"
    url = _http_url(uri)
    opener = opener or urllib.request.urlopen
    offset = 0
    try:
        with open(part, "wb") as f:
            while True:
                req = urllib.request.Request(url, headers={"Range": f"bytes={offset}-{offset + CHUNK - 1}"})
                with opener(req) as r:
                    data = r.read()
                    status = getattr(r, "status", 200)
                f.write(data)
                offset += len(data)
                if status != 206 or len(data) < CHUNK:
                    break
        os.replace(part, dst)
    except Exception as e:
        if os.path.exists(part):
            os.unlink(part)
        raise RuntimeError(f"fetching {redact(uri)} failed: {type(e).__name__}") from None
    return dst
