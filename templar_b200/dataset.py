"""Page-addressed streaming dataset: documents fetched by (config, row offset, split) pages from a rows
service, tokenised, cut at document ends and served as ``[batch, seq_len]`` integer arrays.

Same public surface as the reference's legacy loader (src/tplr/dataset.py:31-186 ``SubsetLoader``,
:189-514 ``DatasetLoader``): ``DatasetLoader.create(...)``, ``next_pages(offset, n_pages, seed)``,
``fetch_dataset_configs()``, ``get_random_pages``, ``get_page_names``, ``fetch_data_to_rows`` and
iteration that yields ``numpy`` batches.  The neurons use the sharded on-disk dataset; this loader is kept
for users that still page a hosted dataset.

Differences in construction, not in behaviour:

* the transport is a small interface (:class:`RowSource`); :class:`HttpRowSource` talks to a
  datasets-server style REST API with ``aiohttp``, :class:`MemoryRowSource` serves documents held in
  memory (tests, air-gapped boxes);
* one ``aiohttp`` session per fetch round, bounded retry with a fixed delay, as the reference;
* documents are kept as separate ``numpy`` arrays in a queue, so building a batch is linear in the
  tokens served instead of re-slicing one long Python list per document.
"""

from __future__ import annotations

import asyncio
import random
from collections import deque
import zlib
from typing import Iterable, Protocol, Sequence

import numpy as np
from torch.utils.data import IterableDataset

Page = tuple[str, int, str]          # (config name, first row, split)


def _seed32(seed) -> int:
    """A 32-bit seed that is the same in every process (the built-in ``hash`` of a string is salted)."""
    if isinstance(seed, (int, np.integer)):
        return int(seed) & 0xFFFFFFFF
    return zlib.crc32(str(seed).encode()) & 0xFFFFFFFF


class RowSource(Protocol):
    async def configs(self) -> dict[str, dict]: ...
    async def rows(self, page: Page, limit: int) -> list[str]: ...


class HttpRowSource:
    """Rows and sizes from a datasets-server style API (``/rows`` and ``/size`` end points)."""

    def __init__(self, name: str, rows_url: str, size_url: str, retry_limit: int = 10, retry_delay: float = 5.0):
        self.name, self.rows_url, self.size_url = name, rows_url, size_url
        self.retry_limit, self.retry_delay = retry_limit, retry_delay
        self._session = None

    async def _get_json(self, url: str, params: dict):
        import aiohttp

        last = None
        for attempt in range(self.retry_limit):
            try:
                session = self._session or aiohttp.ClientSession()
                try:
                    async with session.get(url, params=params) as resp:
                        resp.raise_for_status()
                        return await resp.json()
                finally:
                    if session is not self._session:
                        await session.close()
            except aiohttp.ClientResponseError as e:
                last = e
                if attempt + 1 < self.retry_limit:
                    await asyncio.sleep(self.retry_delay)
        raise RuntimeError(f"Maximum retry attempts exceeded for {url} {params}") from last

    async def __aenter__(self):
        import aiohttp

        self._session = aiohttp.ClientSession()
        return self

    async def __aexit__(self, *exc):
        if self._session is not None:
            await self._session.close()
        self._session = None

    async def configs(self) -> dict[str, dict]:
        data = await self._get_json(self.size_url, {"dataset": self.name})
        return {e["config"]: {"num_rows": e["num_rows"], "split": e["split"]}
                for e in data["size"]["splits"] if e["config"] != "default"}

    async def rows(self, page: Page, limit: int) -> list[str]:
        config, offset, split = page
        data = await self._get_json(self.rows_url, {"dataset": self.name, "config": config, "split": split,
                                                    "offset": offset, "limit": limit})
        return [r["row"]["text"] for r in data["rows"]]


class MemoryRowSource:
    """Documents held in memory: ``{config: [text, ...]}``; every config has one split."""

    def __init__(self, docs: dict[str, Sequence[str]], split: str = "train"):
        self.docs, self.split = docs, split

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc):
        return None

    async def configs(self) -> dict[str, dict]:
        return {c: {"num_rows": len(d), "split": self.split} for c, d in self.docs.items()}

    async def rows(self, page: Page, limit: int) -> list[str]:
        config, offset, _ = page
        return list(self.docs[config][offset: offset + limit])


class SubsetLoader(IterableDataset):
    """Token buffer of fetched documents served as fixed-length sequences.

    Every document ends with the tokenizer's EOS.  Without packing a document is padded with EOS to a
    multiple of ``sequence_length`` (its own EOS dropped first); with ``pack_samples`` documents follow one
    another separated by a single EOS.  Iterating again replays the documents already served before the
    unread ones.  A trailing partial batch is dropped.
    """

    num_rows_per_page = 100

    def __init__(self, batch_size=None, sequence_length=None, num_pages=None, tokenizer=None,
                 pack_samples: bool = False):
        self.batch_size, self.sequence_length, self.num_pages = batch_size, sequence_length, num_pages
        self.tokenizer, self.pack_samples = tokenizer, pack_samples
        self.pages: list[Page] = []
        self._docs: deque[np.ndarray] = deque() # unread documents (EOS-terminated)
        self._used: list[np.ndarray] = []       # documents already cut into sequences
        self._ready = np.zeros(0, dtype=np.int64)
        self.lock = asyncio.Lock()

    # -- views with the reference's attribute names ---------------------------------------- #
    @property
    def buffer(self) -> list[int]:
        return np.concatenate(list(self._docs)).tolist() if self._docs else []

    @property
    def used_buffer(self) -> list[int]:
        return np.concatenate(self._used).tolist() if self._used else []

    @property
    def padded_buffer(self) -> list[int]:
        return self._ready.tolist()

    def add_documents(self, docs: Iterable[Sequence[int]]) -> None:
        """Append tokenised documents; an EOS is added to those that do not end with one."""
        eos = self.tokenizer.eos_token_id
        for d in docs:
            a = np.asarray(d, dtype=np.int64).reshape(-1)
            if a.size == 0 or a[-1] != eos:
                a = np.append(a, eos)
            self._docs.append(a)

    def _get_pad_size(self, input_ids) -> int:
        if self.pack_samples:
            return 1
        return (-len(input_ids)) % self.sequence_length

    def _refill_padded_buffer(self) -> None:
        eos, parts, have = self.tokenizer.eos_token_id, [self._ready], self._ready.size
        while self._docs and have < self.sequence_length:
            doc = self._docs.popleft()
            self._used.append(doc)
            body = doc[:-1]
            pad = self._get_pad_size(body)
            parts += [body, np.full(pad, eos, dtype=np.int64)]
            have += body.size + pad
        if len(parts) > 1:
            self._ready = np.concatenate(parts)

    def __iter__(self):
        self._docs, self._used = deque(self._used + list(self._docs)), []
        self._ready = np.zeros(0, dtype=np.int64)
        self._refill_padded_buffer()
        return self

    def __next__(self) -> np.ndarray:
        batch, L = [], self.sequence_length
        while self._ready.size >= L:
            batch.append(self._ready[:L])
            self._ready = self._ready[L:]
            self._refill_padded_buffer()
            if len(batch) == self.batch_size:
                return np.stack(batch)
        raise StopIteration

    def get_page_names(self) -> list[str]:
        return [f"{cfg}_{row}_{split}" for cfg, row, split in self.pages]


class DatasetLoader(SubsetLoader):
    """Pages of a hosted dataset -> token batches.  ``await DatasetLoader.create(...)`` builds a loaded instance.

    ``source`` (class attribute or ``create(..., source=...)``) is the transport; by default an
    :class:`HttpRowSource` on the class's ``name`` / ``rows_base_url`` / ``size_base_url``.
    """

    name: str = "mlfoundations/dclm-baseline-1.0-parquet"
    rows_base_url: str = "https://datasets-server.huggingface.co/rows"
    size_base_url: str = "https://datasets-server.huggingface.co/size"
    retry_limit: int = 10
    retry_delay: int = 5
    num_rows_per_page: int = 100
    source: RowSource | None = None

    @classmethod
    def _source(cls, source: RowSource | None = None):
        return source or cls.source or HttpRowSource(cls.name, cls.rows_base_url, cls.size_base_url,
                                                     cls.retry_limit, cls.retry_delay)

    def __init__(self, batch_size=None, sequence_length=None, num_pages=None, pages_info=None, tokenizer=None,
                 pack_samples: bool = False, source: RowSource | None = None):
        super().__init__(batch_size, sequence_length, num_pages, tokenizer, pack_samples)
        self.configs_data: dict[str, dict] | None = None
        self._src = self._source(source)

    @classmethod
    async def create(cls, batch_size=None, sequence_length=None, num_pages=None, pages_info=None, tokenizer=None,
                     pack_samples: bool = False, source: RowSource | None = None):
        self = cls(batch_size=batch_size, sequence_length=sequence_length, num_pages=num_pages,
                   tokenizer=tokenizer, pack_samples=pack_samples, source=source)
        self.configs_data = await self._src.configs()
        if pages_info is not None:
            await self._fetch(pages_info)
        elif self.num_pages:
            await self._fetch_data_to_buffer(self.num_pages)
        return self

    # -- page selection --------------------------------------------------------------------- #
    @classmethod
    async def fetch_dataset_configs(cls, source: RowSource | None = None) -> dict[str, dict]:
        """``{config: {"num_rows": n, "split": s}}`` for every config of the dataset except ``default``."""
        return await cls._source(source).configs()

    @classmethod
    async def next_pages(cls, offset: int, n_pages: int, seed, num_rows_per_page: int = 100,
                         source: RowSource | None = None) -> list[Page]:
        """``n_pages`` pages drawn from a generator seeded by ``seed`` and advanced by ``offset`` steps: the
        same (offset, seed) names the same pages on every node (src/tplr/dataset.py:197-213)."""
        configs = await cls.fetch_dataset_configs(source)
        rng = np.random.default_rng(_seed32(seed))
        rng.bit_generator.advance(offset)
        names, out = list(configs.keys()), []
        for _ in range(n_pages):
            cfg = str(rng.choice(names))
            row = int(rng.integers(0, configs[cfg]["num_rows"] - 1 - num_rows_per_page))
            out.append((cfg, row, configs[cfg]["split"]))
        return out

    next_pages_async = next_pages

    def get_random_pages(self, num_pages: int) -> list[Page]:
        pages = []
        for _ in range(num_pages):
            cfg = random.choice(list(self.configs_data.keys()))
            row = random.randint(0, self.configs_data[cfg]["num_rows"] - 1 - self.num_rows_per_page)
            pages.append((cfg, row, self.configs_data[cfg]["split"]))
        return pages

    # -- fetching --------------------------------------------------------------------------- #
    async def _tokenize_content(self, content: str) -> list[int]:
        ids = await asyncio.to_thread(self.tokenizer.encode, content, truncation=True,
                                      max_length=self.sequence_length)
        ids = list(ids)
        ids.append(self.tokenizer.eos_token_id)
        return ids

    async def _page_documents(self, page: Page, src) -> list[list[int]]:
        texts = await src.rows(page, self.num_rows_per_page)
        return list(await asyncio.gather(*[self._tokenize_content(t) for t in texts]))

    async def _fetch_data_for_page(self, page: Page, src=None) -> None:
        docs = await self._page_documents(tuple(page), src or self._src)
        async with self.lock:
            self.add_documents(docs)
            self.pages.append(tuple(page))

    async def _fetch_pages(self, pages: Sequence[Page]) -> None:
        """Fetch all pages concurrently; documents enter the buffer in page order, whatever the arrival order."""
        pages = [tuple(p) for p in pages]
        async with self._src as src:
            per_page = await asyncio.gather(*[self._page_documents(p, src) for p in pages])
        async with self.lock:
            self.pages = []
            self._docs.clear()
            for p, docs in zip(pages, per_page):
                self.add_documents(docs)
                self.pages.append(p)

    async def _fetch(self, page_info: Sequence[Page]) -> None:
        await self._fetch_pages(list(page_info))

    async def fetch_data_for_pages(self, pages: Sequence[Page]) -> None:
        await self._fetch_pages(list(pages))

    async def _fetch_data_to_buffer(self, num_pages: int) -> None:
        await self._fetch_pages(self.get_random_pages(num_pages))

    async def fetch_data_to_rows(self, num_pages: int) -> list[str]:
        """The raw texts of ``num_pages`` random pages (no tokenisation)."""
        async with self._src as src:
            per_page = await asyncio.gather(*[src.rows(p, self.num_rows_per_page)
                                              for p in self.get_random_pages(num_pages)])
        return [t for rows in per_page for t in rows]
