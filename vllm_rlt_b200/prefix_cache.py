"""Prefix reuse over paged KV: complete prompt pages are indexed by a hash chain of their tokens
and mapped into later requests' block tables instead of being recomputed.

The rules are those of the reference's `KVCacheManager` (`vllm_rlt/core/kv_cache_manager.py:219-319`
there):

* the key of page i is `sha256(key of page i - 1 || the page's tokens as little-endian int64)`,
  so a hit on page i implies hits on pages 0..i-1 (`_prefix_keys`, `:219-224`);
* only complete pages are indexed, and never the page holding the last prompt token: the index
  keeps K/V, not the final hidden state the LM head needs, so at least one token is always
  recomputed (`publish_prefix`, `:246-250`; `lookup_prefix` looks up `tokens[:-1]`, `:270`);
* an entry holds one physical page per depth plane (`blocks = tuple(t[index] for t in
  allocation.block_tables)`, `:259`), and every holder of a page counts in its reference count;
* pages with more than one holder are never rolled back (`truncate_suffix` refuses them,
  `:338-356`) — decoding only ever writes behind the prompt, so it never touches them.
"""

from __future__ import annotations

import hashlib
import struct
from collections import OrderedDict


def page_keys(tokens, block: int):
    """Chained digests of the complete pages of `tokens`."""
    digest = b""
    for start in range(0, len(tokens) // block * block, block):
        values = tokens[start:start + block]
        digest = hashlib.sha256(digest + struct.pack(f"<{len(values)}q", *values)).digest()
        yield digest


class PrefixIndex:
    """key -> one physical page per depth plane, in least-recently-used order."""

    def __init__(self, block: int):
        self.block = block
        self._entries: OrderedDict[bytes, tuple[int, ...]] = OrderedDict()
        self.refs: dict[int, int] = {}
        self.queries = 0
        self.hit_tokens = 0

    def __len__(self):
        return len(self._entries)

    def lookup(self, tokens) -> tuple[tuple[int, ...], ...]:
        """Pages (one tuple per page, one id per plane) of the longest indexed prefix of
        `tokens[:-1]`."""
        found = []
        for key in page_keys(tokens[:-1], self.block):
            pages = self._entries.get(key)
            if pages is None:
                break
            self._entries.move_to_end(key)
            found.append(pages)
        return tuple(found)

    def claim(self, prefix) -> None:
        """A request maps `prefix` (a `lookup` result) into its tables."""
        for pages in prefix:
            for b in pages:
                self.refs[b] = self.refs.get(b, 0) + 1
        self.queries += 1
        self.hit_tokens += len(prefix) * self.block

    def publish(self, tokens, length: int, tables) -> int:
        """Index the complete pages of the first `min(length, len(tokens) - 1)` prompt tokens of a
        request whose per-plane block tables are `tables`; returns how many entries were added."""
        added = 0
        publishable = min(length, len(tokens) - 1)
        for index, key in enumerate(page_keys(tokens[:publishable], self.block)):
            if key in self._entries:
                continue
            pages = tuple(int(t[index]) for t in tables)
            for b in pages:
                self.refs[b] = self.refs.get(b, 0) + 1
            self._entries[key] = pages
            added += 1
        return added

    def own(self, blocks) -> None:
        """A request takes fresh pages: it is their first holder."""
        for b in blocks:
            self.refs[int(b)] = self.refs.get(int(b), 0) + 1

    def remap(self, physical) -> None:
        """Rename every page id b to `physical[b]` (ids are dealt in order first and permuted once
        the pool size is known)."""
        self._entries = OrderedDict((k, tuple(physical[b] for b in pages)) for k, pages in self._entries.items())
        self.refs = {physical[b]: n for b, n in self.refs.items()}

    def shared(self, block_id: int) -> bool:
        return self.refs.get(int(block_id), 0) > 1
