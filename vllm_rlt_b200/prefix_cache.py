"""Prefix reuse over paged KV: complete prompt pages are found again by the hash of everything up to
and including them, and mapped into later requests' block tables instead of being recomputed.

The rules are those of the reference's `KVCacheManager` (`vllm_rlt/core/kv_cache_manager.py:219-319`):

* the key of page i is `sha256(key of page i - 1 || the page's tokens as little-endian int64)`, so two
  prompts share a key exactly when they agree on every token up to the end of that page, and the byte
  format is the reference's (a prompt indexed there is found here);
* only complete pages are indexed, and never the page that holds the last prompt token: the index keeps
  K/V, not the hidden state the LM head needs, so the last token is always computed;
* an entry names one physical page per depth plane, and everything that points at a page — the request
  that wrote it, the index, every request that mapped it — counts as a holder;
* a page with more than one holder is never rolled back (`truncate_suffix` refuses, `:338-356`); decoding
  only ever writes behind the prompt, so it never needs to.
"""

from __future__ import annotations

import hashlib
from dataclasses import dataclass


def page_keys(tokens, block: int):
    """One digest per complete page of `tokens`, each chained to the digest before it."""
    previous = b""
    for page in range(len(tokens) // block):
        body = b"".join(int(t).to_bytes(8, "little", signed=True) for t in tokens[page * block:(page + 1) * block])
        previous = hashlib.sha256(previous + body).digest()
        yield previous


@dataclass
class _Entry:
    pages: tuple            # physical page of every depth plane
    touched: int            # value of the index's clock when the entry was last matched or added


class PrefixIndex:
    """digest of a prompt prefix -> the physical pages (one per depth plane) that hold its last page."""

    def __init__(self, block: int):
        self.block = block
        self._entries: dict[bytes, _Entry] = {}
        self._clock = 0
        self.refs: dict[int, int] = {}      # page -> holders
        self.queries = 0
        self.hit_tokens = 0

    def __len__(self):
        return len(self._entries)

    def _tick(self) -> int:
        self._clock += 1
        return self._clock

    def _hold(self, pages) -> None:
        for page in pages:
            page = int(page)
            self.refs[page] = self.refs.get(page, 0) + 1

    def lookup(self, tokens) -> tuple[tuple[int, ...], ...]:
        """The indexed pages a request with this prompt can map: as many leading pages as are both
        complete without the prompt's last token and present in the index (page tuple per page)."""
        reusable = (len(tokens) - 1) // self.block if tokens else 0
        matched = []
        for count, key in enumerate(page_keys(tokens, self.block)):
            entry = self._entries.get(key) if count < reusable else None
            if entry is None:
                break
            entry.touched = self._tick()
            matched.append(entry.pages)
        return tuple(matched)

    def claim(self, prefix) -> None:
        """A request maps the pages of a `lookup` result into its tables and becomes one more holder."""
        self.queries += 1
        self.hit_tokens += self.block * len(prefix)
        for pages in prefix:
            self._hold(pages)

    def own(self, pages) -> None:
        """A request takes fresh pages of its own: their first holder."""
        self._hold(pages)

    def publish(self, tokens, computed: int, tables) -> int:
        """Offers a request's prompt pages to later requests.  `computed` prompt tokens are in the cache
        and `tables[plane][page]` are the request's pages; every complete page that lies before the last
        prompt token and is not indexed yet gets an entry (and the index as a holder).  Returns how many."""
        usable = min(computed, len(tokens) - 1) // self.block
        fresh = 0
        for page, key in enumerate(page_keys(tokens, self.block)):
            if page >= usable:
                break
            if key not in self._entries:
                pages = tuple(int(plane[page]) for plane in tables)
                self._entries[key] = _Entry(pages, self._tick())
                self._hold(pages)
                fresh += 1
        return fresh

    def remap(self, physical) -> None:
        """Renames every page id b to `physical[b]` (ids are dealt in order first and shuffled once the pool
        size is known)."""
        for entry in self._entries.values():
            entry.pages = tuple(physical[b] for b in entry.pages)
        self.refs = {physical[b]: holders for b, holders in self.refs.items()}

    def shared(self, page: int) -> bool:
        return self.refs.get(int(page), 0) > 1

    def least_recent(self):
        """Digest of the entry matched longest ago (the one an eviction would drop first), or None."""
        return min(self._entries, key=lambda key: self._entries[key].touched, default=None)
