"""Native tokenizer, safetensors reader and the Hugging Face -> weight-segment converter (CPU)."""
import ctypes
import json

import pytest
import torch

from blitz_scale_b200.runtime import core

CORPUS = ["The quick brown fox jumps over the lazy dog. " * 3,
          "Hello, world! It's 2024 and we're testing tokenizers: 12345 67 8.",
          "def foo(x):\n    return x + 1\n\n# comment   with   spaces",
          "naïve café — ünïcödé ✓ 日本語"] * 5
PROBES = CORPUS[:4] + ["  leading spaces", "tabs\tand\nnewlines\n\n  x", "<|begin|>hi there<|end|>",
                       "it's we'll I'd 'quoted'", "a1b22c333d4444", "end with space ", "x  y   z", ""]


@pytest.fixture(scope="module")
def trained(tmp_path_factory):
    tk = pytest.importorskip("tokenizers")
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers, trainers
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    tok.decoder = decoders.ByteLevel()
    tr = trainers.BpeTrainer(vocab_size=600, special_tokens=["<|begin|>", "<|end|>"],
                             initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(CORPUS, tr)
    p = str(tmp_path_factory.mktemp("tok") / "tokenizer.json")
    tok.save(p)
    return tok, p


def test_byte_level_bpe_matches_reference_library(trained):
    """Same ids as the Hugging Face `tokenizers` library on the same tokenizer.json; lossless round trip."""
    ref, path = trained
    t = core.Tokenizer.from_file(path)
    assert t.num_ids() == ref.get_vocab_size()
    for s in PROBES:
        ids = t.encode(s)
        assert ids == ref.encode(s).ids, s
        assert t.decode(ids, False) == s
    assert t.decode(t.encode("<|begin|>hi<|end|>"), True) == "hi"
    assert t.get_id("<|end|>") == ref.token_to_id("<|end|>") and t.get_id("no such token") == -1
    assert t.is_special(t.get_id("<|end|>")) and not t.is_special(t.get_id("a")) and not t.is_special(-1) and not t.is_special(10 ** 6)
    # ids that a model may emit in any order: bytes that form no character decode to U+FFFD, as in the library
    import random
    rng = random.Random(5)
    lossy = 0
    for _ in range(200):
        ids = [rng.randrange(t.num_ids()) for _ in range(rng.randrange(1, 6))]
        got = t.decode(ids, True)
        assert got == ref.decode(ids, skip_special_tokens=True), ids
        lossy += "\ufffd" in got
    assert lossy > 0
    assert t.decode_bytes(t.encode("é")[:1], True) in ("é".encode(), "é".encode()[:1])


def test_concurrent_encodes_share_the_word_cache_safely(trained):
    """`encode` releases the interpreter lock and the router calls it from several threads: the shared word cache must
    give every thread the ids a single thread gets."""
    import random
    from concurrent.futures import ThreadPoolExecutor
    ref, path = trained
    t = core.Tokenizer.from_file(path)
    rng = random.Random(4)
    words = ["hello", "world", "tokenizer", "naïve", "日本語", "123", "don't", "  ", "\n", "x" * 300]
    texts = [" ".join(rng.choice(words) + str(rng.randrange(50)) for _ in range(200)) for _ in range(64)]
    want = [ref.encode(x).ids for x in texts]
    with ThreadPoolExecutor(max_workers=8) as ex:
        for _ in range(3):
            assert list(ex.map(t.encode, texts)) == want


def test_tokenizer_c_abi(trained):
    _, path = trained
    lib = ctypes.CDLL(core._m.__file__)     # the C ABI lives in the same shared object as the Python module
    lib.blitz_tokenizer_create_from_file.restype = ctypes.c_void_p
    lib.blitz_tokenizer_encode.restype = ctypes.c_int64
    lib.blitz_tokenizer_decode.restype = ctypes.c_int64
    h = ctypes.c_void_p(lib.blitz_tokenizer_create_from_file(path.encode()))
    assert h.value
    text = "Hello, world! 123".encode()
    buf = (ctypes.c_int32 * 64)()
    n = lib.blitz_tokenizer_encode(h, text, ctypes.c_int64(len(text)), buf, ctypes.c_int64(64))
    assert 0 < n <= 64 and list(buf[:n]) == core.Tokenizer.from_file(path).encode(text.decode())
    out = ctypes.create_string_buffer(256)
    m = lib.blitz_tokenizer_decode(h, buf, ctypes.c_int64(n), 1, out, ctypes.c_int64(256))
    assert out.raw[:m] == text
    assert lib.blitz_tokenizer_num_ids(h) > 256
    lib.blitz_tokenizer_free(h)
    assert lib.blitz_tokenizer_create_from_file(b"/nonexistent/tokenizer.json") is None


def test_sentencepiece_style_bpe_with_byte_fallback():
    vocab = {"<unk>": 0, "<s>": 1, "</s>": 2}
    for b in range(256):
        vocab[f"<0x{b:02X}>"] = 3 + b
    for i, tok in enumerate(["▁", "h", "e", "l", "o", "w", "r", "d", "he", "ll", "hell", "hello", "▁hello",
                             "▁w", "or", "▁wor", "ld", "▁world"]):
        vocab[tok] = 259 + i
    merges = ["h e", "l l", "he ll", "hell o", "▁ hello", "▁ w", "o r", "▁w or", "l d", "▁wor ld"]
    js = {"model": {"type": "BPE", "vocab": vocab, "merges": merges, "byte_fallback": True, "unk_token": "<unk>"},
          "normalizer": {"type": "Sequence"}, "pre_tokenizer": None, "decoder": {"type": "Sequence"},
          "added_tokens": [{"id": 1, "content": "<s>", "special": True}, {"id": 2, "content": "</s>", "special": True}]}
    t = core.Tokenizer.from_json(json.dumps(js))
    ids = t.encode("hello world")
    assert ids == [vocab["▁hello"], vocab["▁world"]]
    assert t.decode(ids) == "hello world"
    z = t.encode("hello Z")       # 'Z' is not in the vocabulary -> byte token
    assert z[-1] == vocab["<0x5A>"] and t.decode(z) == "hello Z"
    assert t.encode("<s>hello")[0] == 1
    # a damaged file: an id far beyond any vocabulary is refused instead of sizing the id table
    for broken in ({**js, "model": {**js["model"], "vocab": {**vocab, "zz": 99999999999}}},
                   {**js, "added_tokens": [{"id": 2 ** 40, "content": "<x>", "special": True}]}):
        with pytest.raises(RuntimeError):
            core.Tokenizer.from_json(json.dumps(broken))
    # this family merges a whole prompt as one piece: the merge loop must not be quadratic in its length
    import time
    long_text = "hello world " * 20000                       # 240 k characters
    t0 = time.perf_counter()
    ids = t.encode(long_text)
    assert time.perf_counter() - t0 < 5.0
    # the trailing space becomes a "▁" of its own, which this toy vocabulary holds
    assert ids[:2] == [vocab["▁hello"], vocab["▁world"]] and len(ids) == 40001 and ids[-1] == vocab["▁"]


def test_one_very_long_word_is_tokenized_in_near_linear_time(trained):
    """A run of one letter is a single word for the pre-tokenizer; its cost must stay near linear (a quadratic merge
    loop needs minutes for this input) and the ids are the reference library's."""
    import time
    ref, path = trained
    t = core.Tokenizer.from_file(path)
    for text in ("a" * 20000, "ab" * 10000, "the" * 7000):
        assert t.encode(text) == ref.encode(text).ids
    t0 = time.perf_counter()
    n = len(t.encode("a" * 400000))
    assert n > 0 and time.perf_counter() - t0 < 5.0


def test_safetensors_reader_and_hf_conversion(tmp_path):
    from blitz_scale_b200.models import convert
    from blitz_scale_b200.models.config import get_config
    from blitz_scale_b200.models.weights import WeightSegment, shard_from_full
    cfg = get_config("tiny")
    seg = WeightSegment(cfg, dtype=torch.bfloat16).random_init_(seed=3)
    hf = convert.segment_to_hf(seg)
    # two shard files, like a real checkpoint
    names = list(hf)
    convert.write_safetensors(tmp_path / "model-00001-of-00002.safetensors", {n: hf[n] for n in names[:5]}, {"format": "pt"})
    convert.write_safetensors(tmp_path / "model-00002-of-00002.safetensors", {n: hf[n] for n in names[5:]})
    f = core.SafeTensorsFile(str(tmp_path / "model-00001-of-00002.safetensors"))
    assert f.metadata() == [("format", "pt")] and f.names() == names[:5]
    info = f.info("model.embed_tokens.weight")
    assert info.dtype == "BF16" and list(info.shape) == [cfg.vocab, cfg.hidden] and info.nbytes == cfg.vocab * cfg.hidden * 2
    with pytest.raises(KeyError):
        f.info("missing")
    # a header whose numbers do not describe bytes of the file is refused, whatever they would wrap to
    import json
    import struct
    for entry in ({"dtype": "WEIRD", "shape": [1], "data_offsets": [0, 1.8e19]}, {"dtype": "F32", "shape": [2], "data_offsets": [-8, 0]},
                  {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}, {"dtype": "F32", "shape": [2 ** 62, 4], "data_offsets": [0, 8]},
                  {"dtype": "F32", "shape": [2], "data_offsets": [0, 1e300]}, {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}):
        hb = json.dumps({"t": entry}).encode()
        bad = tmp_path / "bad.bin"
        bad.write_bytes(struct.pack("<Q", len(hb)) + hb + bytes(16))
        with pytest.raises(RuntimeError):
            core.SafeTensorsFile(str(bad))
    bad.write_bytes(struct.pack("<Q", 2 ** 63) + b"{}")
    with pytest.raises(RuntimeError):
        core.SafeTensorsFile(str(bad))
    back = convert.hf_to_segment(convert.CheckpointReader(tmp_path), cfg)
    assert torch.equal(back.buffer, seg.buffer)             # byte-exact round trip through HF names and layout
    paths = convert.convert(tmp_path, "tiny", tmp_path / "out", tp=2)
    assert len(paths) == 2
    for r, p in enumerate(paths):
        want = shard_from_full(seg, 2, r, device="cpu")
        got = torch.from_file(str(p), size=want.layout.total_bytes, dtype=torch.uint8)
        assert torch.equal(got, want.buffer[:want.layout.total_bytes])
        WeightSegment.check_sidecar(p.parent, cfg, 2, r, torch.bfloat16)
    assert convert.main(["--src", str(tmp_path), "--model", "tiny", "--out", str(tmp_path / "cli")]) == 0
    assert (tmp_path / "cli" / "segment.0.bin").stat().st_size == seg.layout.total_bytes
    # scalars, integer and boolean tensors, empty tensors: both directions against the `safetensors` library
    st_lib = pytest.importorskip("safetensors.torch")
    odd = {"scalar": torch.tensor(2.5), "ids": torch.arange(6, dtype=torch.int64).view(2, 3), "mask": torch.tensor([True, False]),
           "empty": torch.zeros(0, 4, dtype=torch.float16), "bytes": torch.arange(5, dtype=torch.uint8)}
    st_lib.save_file(odd, str(tmp_path / "odd.safetensors"))
    r = convert.CheckpointReader(tmp_path / "odd.safetensors")
    for k, v in odd.items():
        got = r.get(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v), k
    convert.write_safetensors(tmp_path / "odd2.safetensors", odd)
    back = st_lib.load_file(str(tmp_path / "odd2.safetensors"))
    assert all(back[k].dtype == v.dtype and back[k].shape == v.shape and torch.equal(back[k], v) for k, v in odd.items())
    (tmp_path / "odd.safetensors").unlink()
    (tmp_path / "odd2.safetensors").unlink()
    # list and verify modes
    listed = convert.list_checkpoint(tmp_path)
    assert ("lm_head.weight", "BF16", (cfg.vocab, cfg.hidden)) in listed and len(listed) == 3 + 9 * cfg.layers
    assert convert.main(["--src", str(tmp_path), "--list"]) == 0
    assert convert.verify(tmp_path, "tiny", tmp_path / "out", tp=2) == []
    assert convert.main(["--src", str(tmp_path), "--model", "tiny", "--out", str(tmp_path / "out"), "--tp", "2", "--verify"]) == 0
    with open(paths[1], "r+b") as f:                       # flip one byte inside rank 1's first layer
        f.seek(WeightSegment(cfg, 2, 1, device="meta").layout.unit("layer.0")[0] + 64)
        b = f.read(1)
        f.seek(-1, 1)
        f.write(bytes([b[0] ^ 0x40]))
    bad = convert.verify(tmp_path, "tiny", tmp_path / "out", tp=2)
    assert len(bad) == 1 and bad[0].startswith("rank 1: layers.0.")
    assert convert.main(["--src", str(tmp_path), "--model", "tiny", "--out", str(tmp_path / "out"), "--tp", "2", "--verify"]) == 1
    # a truncated file is rejected, not mis-read
    raw = (tmp_path / "model-00002-of-00002.safetensors").read_bytes()
    (tmp_path / "bad.safetensors").write_bytes(raw[:len(raw) // 2])
    with pytest.raises(RuntimeError):
        core.SafeTensorsFile(str(tmp_path / "bad.safetensors"))


def test_native_logger_and_contracts(tmp_path):
    import subprocess
    import sys
    code = ("from blitz_scale_b200.runtime import core\n"
            "core.native_log(2, 'hello info'); core.native_log(1, 'hidden debug'); core.native_log(4, 'bad thing')\n"
            "assert core.native_log_enabled(2) and not core.native_log_enabled(1)\n"
            "core.set_native_log_level('trace'); core.native_log(0, 'now visible')\n"
            "core.check_precondition(True)\n"
            "try:\n    core.check_precondition(False)\n    raise SystemExit(3)\nexcept RuntimeError as e:\n    assert 'precondition failed: ok' in str(e)\n")
    logf = tmp_path / "rank0.log"
    env = dict(__import__("os").environ, BLITZ_LOG_FILE=str(logf), LOG_LEVEL="info")
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    text = logf.read_text()
    assert "INFO  python:0 hello info" in text and "hidden debug" not in text and "ERROR python:0 bad thing" in text
    assert "TRACE python:0 now visible" in text and "precondition failed" in text


def test_router_http_with_native_tokenizer(trained):
    """Text in -> native tokenizer -> generation -> text out, over the HTTP API against a stub worker."""
    import asyncio
    import socket

    import aiohttp

    from blitz_scale_b200.router.runtime import RouterRuntime
    from blitz_scale_b200.router.server import controller_config_from_cluster, serve_router
    from blitz_scale_b200.sim.stub_worker import StubBackend
    from blitz_scale_b200.worker.service import serve
    ref, path = trained
    socks = [socket.socket() for _ in range(2)]
    for s_ in socks:
        s_.bind(("127.0.0.1", 0))
    wport, hport = [s_.getsockname()[1] for s_ in socks]
    for s_ in socks:
        s_.close()

    async def go():
        stop, ready = asyncio.Event(), asyncio.Event()
        b = StubBackend(0, 1, vocab=ref.get_vocab_size())
        tasks = [asyncio.create_task(serve(b, "127.0.0.1", wport, stop_event=stop, ready_event=ready))]
        await ready.wait()
        cfg = controller_config_from_cluster({"init_states": ["Normal"], "machines": [0]}, 1, "impl_blitz,manually_scale",
                                             max_blocks_per_replica=4000)
        rt = RouterRuntime(cfg, [f"127.0.0.1:{wport}"], model_layers=2)
        tasks.append(asyncio.create_task(serve_router(rt, "127.0.0.1", hport, stop=stop, model_name="tiny",
                                                      tokenizer_path=path, tokenizer_workers=2)))
        await asyncio.sleep(0.3)
        text = "Hello, world! It's 2024 and we're testing tokenizers."
        async with aiohttp.ClientSession() as s:
            async with s.post(f"http://127.0.0.1:{hport}/generate",
                              json={"inputs": text, "parameters": {"max_new_tokens": 5, "details": True}}) as r:
                assert r.status == 200, await r.text()
                body = await r.json()
                hdr = dict(r.headers)
            async with s.post(f"http://127.0.0.1:{hport}/generate", json={"input_tokens": [10 ** 6], "parameters": {}}) as r:
                assert r.status == 422 and "input_tokens" in (await r.json())["error"]
            # a stop sequence in real text: the text that the third token of the next request adds ends the request
            # there (the stub's tokens are a function of the request id and the position)
            from blitz_scale_b200.sim.stub_worker import stub_token
            import re
            t = core.Tokenizer.from_file(path)
            stopped = None
            for extra in range(40):                      # a prompt whose (random) continuation contains a clean word
                prompt = text + " a" * extra
                n_in = len(t.encode(prompt))
                exp = [stub_token(0, rt._next_id, n_in + n, ref.get_vocab_size()) for n in range(8)]
                words = re.findall(r"[A-Za-z]{2,}", t.decode(exp, True))
                cuts = [(next(k for k in range(1, 9) if w in t.decode(exp[:k], True)), w) for w in words]
                cuts = [c for c in cuts if 2 <= c[0] < 8]
                if not cuts:
                    continue
                cut, word = min(cuts)
                async with s.post(f"http://127.0.0.1:{hport}/generate",
                                  json={"inputs": prompt, "parameters": {"max_new_tokens": 8, "details": True, "stop": [word],
                                                                         "return_full_text": True}}) as r:
                    assert r.status == 200, await r.text()
                    stopped = (await r.json(), exp[:cut], prompt + t.decode(exp[:cut], True))
                break
        stop.set()
        await asyncio.wait(tasks, timeout=5)
        return text, body, hdr, stopped

    text, body, hdr, stopped = asyncio.run(go())
    assert stopped is not None
    got, want_ids, want_text = stopped
    assert [tk["id"] for tk in got["details"]["tokens"]] == want_ids and got["details"]["finish_reason"] == "stop_sequence"
    assert got["generated_text"] == want_text
    assert body["details"]["finish_reason"] == "length"
    t = core.Tokenizer.from_file(path)
    assert int(hdr["x-input-length"]) == len(t.encode(text)) == len(ref.encode(text).ids)
    ids = [tk["id"] for tk in body["details"]["tokens"]]
    assert len(ids) == 5 and body["generated_text"] == t.decode(ids, True)
    assert [tk["text"] for tk in body["details"]["tokens"]] == [t.decode([i], False) for i in ids]


LLAMA3_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+"
                  r"|\s+(?!\S)|\s+")
QWEN2_PATTERN = LLAMA3_PATTERN.replace(r"\p{N}{1,3}", r"\p{N}")
HARD = ["word—word ² ³ ١٢٣ 12345 x1y22z333", "tab\there\r\nnext  line\n\n  indented", "I'M HE'LL we'Ve 'quoted' don't",
        "naïve café — ünïcödé ✓ 日本語 한국어 😀😀", "a b c 　d  e", "price: $1,234.56 (approx.)!!!\n",
        "foo_bar-baz/qux.py:42", "  a", "x \n\n y\r\n\r\n  z  "]


@pytest.mark.parametrize("kind", ["gpt2", "llama3", "qwen2"])
def test_word_patterns_match_the_reference_library_on_random_text(kind, tmp_path):
    """Token ids equal those of the `tokenizers` library for GPT-2's word pattern and for the cl100k-family patterns of
    Llama-3 and Qwen-2 (a Split pre-tokenizer in tokenizer.json), on hand-picked hard cases and on random strings
    rich in Unicode white space, digits and punctuation."""
    pytest.importorskip("tokenizers")
    hypothesis = pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    from tokenizers import Regex, Tokenizer, decoders, models, pre_tokenizers, trainers
    ref = Tokenizer(models.BPE())
    if kind == "gpt2":
        ref.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=True)
    else:
        pat = LLAMA3_PATTERN if kind == "llama3" else QWEN2_PATTERN
        ref.pre_tokenizer = pre_tokenizers.Sequence([pre_tokenizers.Split(Regex(pat), behavior="isolated", invert=False),
                                                     pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    ref.decoder = decoders.ByteLevel()
    ref.train_from_iterator(CORPUS + HARD * 4, trainers.BpeTrainer(vocab_size=900, special_tokens=["<|begin|>", "<|end|>"],
                                                                   initial_alphabet=pre_tokenizers.ByteLevel.alphabet(),
                                                                   show_progress=False))
    ref.save(str(tmp_path / "tokenizer.json"))
    nat = core.Tokenizer.from_file(str(tmp_path / "tokenizer.json"))
    for s in HARD + PROBES:
        assert nat.encode(s) == ref.encode(s).ids, (kind, s)
        assert nat.decode(nat.encode(s), False) == s
    if kind != "gpt2":
        assert nat.encode("in 12345 days") != core.Tokenizer.from_file(str(tmp_path / "tokenizer.json")).encode("in 12 345 days")
    pieces = st.sampled_from(list("abcXYZ019 '\t\n\r.,!?-_’é日本ñ²١—✓😀$") + ["'s", "'LL", "'Ve", " ", " ", "　",
                                                                              "  ", "\r\n", "<|end|>", "12345", " the", "word"])

    @settings(max_examples=400, deadline=None)
    @given(st.lists(pieces, max_size=20).map("".join))
    def agree(s):
        ids = nat.encode(s)
        assert ids == ref.encode(s).ids, (kind, s)
        assert nat.decode(ids, False) == s
    agree()


def test_sentencepiece_style_matches_the_reference_library_on_random_text(tmp_path):
    pytest.importorskip("tokenizers")
    pytest.importorskip("hypothesis")
    from hypothesis import given, settings, strategies as st
    from tokenizers import Tokenizer, decoders, models, normalizers, trainers
    ref = Tokenizer(models.BPE(unk_token="<unk>", byte_fallback=True, fuse_unk=True))
    ref.normalizer = normalizers.Sequence([normalizers.Prepend("▁"), normalizers.Replace(" ", "▁")])
    ref.decoder = decoders.Sequence([decoders.Replace("▁", " "), decoders.ByteFallback(), decoders.Fuse(), decoders.Strip(" ", 1, 0)])
    ref.train_from_iterator(CORPUS, trainers.BpeTrainer(vocab_size=700, show_progress=False,
                                                        special_tokens=["<unk>", "<s>", "</s>"] + [f"<0x{i:02X}>" for i in range(256)]))
    ref.save(str(tmp_path / "tokenizer.json"))
    nat = core.Tokenizer.from_file(str(tmp_path / "tokenizer.json"))
    pieces = st.sampled_from(list("abcXYZ019 '\t\n.,!?-_é日ñ—😀") + [" ", "  ", "the", " quick", "<s>", "</s>", "▁"])

    @settings(max_examples=400, deadline=None)
    @given(st.lists(pieces, max_size=20).map("".join))
    def agree(s):
        ids = nat.encode(s)
        assert ids == ref.encode(s).ids, s
        assert nat.decode(ids, True) == ref.decode(ids, skip_special_tokens=True), s
    agree()
