"""MetaServer and its client against a real aiohttp server on an ephemeral port:
every route, objects, sets, barriers, waits and their timeouts, keys with
slashes, the id allocator, and failure behaviour (dropped keys, a server that is
gone, a rank that never joins)."""

import threading
import time

import pytest
import requests

from awex_b200.meta.meta_server import MetaServer, MetaServerClient
from awex_b200.utils.common import from_binary, to_binary


@pytest.fixture()
def served():
    server = MetaServer("127.0.0.1", 0)
    server.start()
    client = MetaServerClient("127.0.0.1", server.port, max_retries=2)
    yield server, client
    client.close()
    server.stop()


def test_store_api_without_http():
    server = MetaServer("127.0.0.1", 0)
    server.put_object("a", {"x": 1})
    assert server.get_object("a") == {"x": 1}
    server.put_binary("b", b"raw")
    assert server.get_binary("b") == b"raw"
    server.put_json("j", [1, 2])
    assert server.get_json("j") == [1, 2]
    server.delete("a")
    with pytest.raises(Exception):
        server.get_binary("a")


def test_raw_routes(served):
    server, _ = served
    base = f"http://127.0.0.1:{server.port}/v1"
    assert requests.get(f"{base}/health").json()["success"]
    assert requests.get(f"{base}/get_binary/missing").status_code == 404
    assert requests.put(f"{base}/put_binary/k", data=b"\x00\x01").json()["success"]
    assert requests.get(f"{base}/get_binary/k").content == b"\x00\x01"
    assert requests.get(f"{base}/has_key/k").json()["has_key"] is True
    assert requests.get(f"{base}/has_key/other").json()["has_key"] is False
    assert "k" in requests.get(f"{base}/keys").json()["keys"]
    assert requests.put(f"{base}/put_json/doc", json={"a": [1, 2]}).json()["success"]
    assert requests.get(f"{base}/get_json/doc").json()["data"] == {"a": [1, 2]}
    assert requests.get(f"{base}/get_json/nodoc").status_code == 404
    assert requests.put(f"{base}/add_object_to_set/s", data=to_binary(3)).json()["success"]
    assert requests.put(f"{base}/add_object_to_set/s", data=to_binary(3)).json()["success"]
    assert from_binary(requests.get(f"{base}/get_binary/s").content) == {3}
    assert requests.delete(f"{base}/delete/k").json()["success"]
    assert requests.delete(f"{base}/delete/k").status_code == 404
    first = requests.post(f"{base}/allocate_auto_grow_id").json()["id"]
    assert requests.post(f"{base}/allocate_auto_grow_id").json()["id"] == first + 1


def test_client_objects_sets_and_slash_keys(served):
    _, c = served
    c.put_object("step/1/meta", {"names": ["a", "b"], "n": 2})
    assert c.get_object("step/1/meta") == {"names": ["a", "b"], "n": 2}
    assert c.has_key("step/1/meta") and "step/1/meta" in c.list_keys()
    assert c.get_object("absent") is None
    assert c.get_object("absent", default_value=7) == 7
    with pytest.raises(ValueError):
        c.get_binary("absent")
    c.put_binary("blob", b"abc")
    assert c.get_binary("blob") == b"abc"
    c.put_json("cfg", {"tp": 2})
    assert c.get_json("cfg") == {"tp": 2}
    with pytest.raises(ValueError):
        c.get_json("nocfg")
    for r in (0, 1, 1, 2):
        c.add_object_to_set("joined", r)
    assert c.get_set("joined") == {0, 1, 2} and c.get_set("nobody") == set()
    c.put_object("once", (1, 2))
    assert c.get_object_then_delete("once", timeout=1) == (1, 2) and not c.has_key("once")
    c.delete_if_exists("once")  # absent keys are fine
    a, b = c.allocate_auto_grow_id(), c.allocate_auto_grow_id()
    assert b == a + 1
    assert c.health_check()["success"]


def test_waits_return_when_posted_and_time_out_when_not(served):
    _, c = served
    threading.Timer(0.3, lambda: MetaServerClient("127.0.0.1", c._port).put_object("late", 5)).start()
    started = time.time()
    assert c.get_object("late", timeout=10) == 5
    assert time.time() - started < 5
    started = time.time()
    with pytest.raises(TimeoutError):
        c.wait_key("never", timeout=0.5)
    assert time.time() - started < 3
    assert c.get_object("never", timeout=0.3, default_value="fallback") == "fallback"
    with pytest.raises(TimeoutError):
        c.get_object("never", timeout=0.3)


def test_barrier_completes_and_a_missing_rank_times_out(served):
    _, c = served
    port = c._port
    done = []

    def member(rank):
        MetaServerClient("127.0.0.1", port).barrier("b1", rank, 3, timeout=20)
        done.append(rank)

    threads = [threading.Thread(target=member, args=(r,)) for r in range(3)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
    assert sorted(done) == [0, 1, 2]
    # rank 2 never joins: the others give up after their timeout instead of hanging
    with pytest.raises(TimeoutError):
        c.barrier("b2", 0, 3, timeout=0.6)
    c.add_object_to_set("grow", 1)
    with pytest.raises(TimeoutError):
        c.wait_set_until_size("grow", 2, timeout=0.5)
    c.add_object_to_set("grow", 2)
    c.wait_set_until_size("grow", 2, timeout=5, delete_after_wait=True)
    assert not c.has_key("grow")


def test_client_gives_up_when_the_server_is_gone():
    server = MetaServer("127.0.0.1", 0)
    server.start()
    port = server.port
    c = MetaServerClient("127.0.0.1", port, max_retries=1)
    c.put_object("x", 1)
    server.stop()
    with pytest.raises(Exception):
        c.put_object("y", 2)
    c.delete_if_exists("x")  # swallowed


def test_counters_wake_waiters_without_polling(served):
    """`put_counter` / `wait_counters`: a waiter sleeps inside the server and is
    answered when the last counter it names reaches the value; a wait that cannot
    be satisfied ends with the host-handshake timeout of the data plane."""
    import threading

    from awex_b200.transfer.transports import HostHandshakeTimeout, done_key, launched_key, ready_key, wait_counters

    _, c = served
    assert ready_key(3) == "p2p_ready_3" and launched_key(9) == "p2p_launched_9" and done_key(9) == "p2p_done_9"
    assert c.get_counter(ready_key(0)) is None
    started = time.time()
    with pytest.raises(HostHandshakeTimeout):
        wait_counters(c, [ready_key(0)], 1, timeout_s=0.2)
    assert time.time() - started < 2
    c.put_counter(ready_key(0), [1, 5])
    assert wait_counters(c, [ready_key(0)], 1, timeout_s=0.2) == {ready_key(0): [1, 5]}
    with pytest.raises(HostHandshakeTimeout):  # epoch 1 is there, epoch 2 is not
        wait_counters(c, [ready_key(0)], 2, timeout_s=0.2)
    # two counters, the second arrives while the request sleeps in the server
    other = MetaServerClient("127.0.0.1", c._port)
    timer = threading.Timer(0.3, lambda: other.put_counter(ready_key(1), 4))
    timer.start()
    started = time.time()
    got = wait_counters(c, [ready_key(0), ready_key(1)], 1, timeout_s=10)
    waited = time.time() - started
    timer.join()
    assert got == {ready_key(0): [1, 5], ready_key(1): [4]} and 0.2 < waited < 3
    c.put_counter("odd/key with spaces", 7)  # keys are quoted on the wire
    assert c.get_counter("odd/key with spaces") == [7]


@pytest.mark.timeout(180)
def test_server_in_a_subprocess_starts_answers_and_stops():
    """`start_meta_server` spawns the server in a daemon subprocess (with an
    empty host it picks this machine's address), returns where it listens, and
    `stop_meta_server` reaps it."""
    from awex_b200.meta.meta_server import MetaServerClient, start_meta_server, stop_meta_server

    address, port = start_meta_server("127.0.0.1", 0)
    try:
        assert address == "127.0.0.1" and port > 0
        client = MetaServerClient(address, port)
        assert client.health_check()
        client.put_object("k", {"a": 1})
        client.put_binary("b", b"\x00\x01")
        client.add_object_to_set("s", 3)
        assert client.get_object("k", timeout=5) == {"a": 1}
        # one delete route for every kind of value
        for key in ("k", "b", "s"):
            assert client.has_key(key)
            client.delete(key)
            assert not client.has_key(key)
    finally:
        assert stop_meta_server() is True
    assert stop_meta_server() is False  # nothing left to stop


def test_optional_shared_secret(monkeypatch):
    """With AWEX_META_SERVER_TOKEN set, requests without the secret are refused
    (the health probe stays open); clients created with it in their environment
    work as before."""
    import requests

    from awex_b200.meta.meta_server import MetaServer, MetaServerClient

    monkeypatch.setenv("AWEX_META_SERVER_TOKEN", "s3cret")
    server = MetaServer("127.0.0.1", 0)
    server.start()
    try:
        base = f"http://127.0.0.1:{server.port}/v1"
        assert requests.get(f"{base}/health").status_code == 200
        assert requests.put(f"{base}/put_binary/k", data=b"x").status_code == 401
        assert requests.get(f"{base}/keys").status_code == 401
        assert requests.get(f"{base}/keys", headers={"X-Awex-Token": "wrong"}).status_code == 401
        client = MetaServerClient("127.0.0.1", server.port)
        client.put_object("k", [1, 2])
        assert client.get_object("k", timeout=5) == [1, 2] and client.list_keys() == ["k"]
        monkeypatch.delenv("AWEX_META_SERVER_TOKEN")
        stranger = MetaServerClient("127.0.0.1", server.port, max_retries=1)
        monkeypatch.setenv("AWEX_META_SERVER_TOKEN", "s3cret")  # the server still has it; the stranger's session was made without
        with pytest.raises(requests.HTTPError, match="401"):
            stranger.has_key("k")
    finally:
        server.stop()
