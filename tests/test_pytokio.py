"""Tasks on the native runtime (PythonTask / Shared) and the event-loop integration of
endpoint futures.  Modelled on the reference's pytokio usage (python/tests/test_future.py,
test_python_actors.py async sections)."""
import asyncio
import threading
import time

import pytest

from monarch_b200 import _native as N
from monarch_b200.actor import Actor, endpoint, this_host
from monarch_b200.actor.future import Future, FutureTimeout, select_one
from monarch_b200.actor.pytokio import PythonTask, Shared, is_tokio_thread


def test_tasks_block_spawn_and_share():
    assert PythonTask(lambda: 6 * 7).block_on() == 42
    sh = PythonTask(lambda: threading.current_thread().name).spawn()
    assert isinstance(sh, Shared)
    assert sh.block_on() == sh.block_on()           # the result can be taken repeatedly
    assert sh.task().block_on() == sh.block_on()
    t = PythonTask(lambda: 1)
    t.spawn()
    with pytest.raises(RuntimeError, match="once"):
        t.spawn()
    with pytest.raises(ZeroDivisionError):
        PythonTask(lambda: 1 // 0).block_on()
    assert not is_tokio_thread()
    assert PythonTask.spawn_blocking(is_tokio_thread).block_on() is True


def test_coroutines_await_tasks_without_an_event_loop():
    async def leaf(x):
        return await PythonTask(lambda: x + 1)

    async def tree():
        a = PythonTask.from_coroutine(leaf(1)).spawn()
        b = PythonTask.from_coroutine(leaf(10)).spawn()
        return (await a) + (await b) + (await a)       # a Shared is awaitable repeatedly

    assert PythonTask.from_coroutine(tree()).block_on() == 2 + 11 + 2

    async def failing():
        try:
            await PythonTask(lambda: 1 // 0)
        except ZeroDivisionError:
            return "caught"
    assert PythonTask.from_coroutine(failing()).block_on() == "caught"

    async def wrong():
        await asyncio.sleep(0)           # not a pytokio awaitable
    with pytest.raises((TypeError, RuntimeError)):
        PythonTask.from_coroutine(wrong()).block_on()


def test_many_waiting_coroutines_park_no_threads():
    gate = N.Completion()

    async def waiter(i):
        return i + await Shared(gate)

    before = N.task_pool_threads()
    tasks = [PythonTask.from_coroutine(waiter(i)).spawn() for i in range(200)]
    time.sleep(0.2)
    assert N.task_pool_threads() - before <= 8       # suspended, not blocked
    gate.set_result(1000)
    assert [t.block_on(10) for t in tasks] == [1000 + i for i in range(200)]


def test_with_timeout_and_select_one():
    slow = PythonTask(lambda: time.sleep(5) or "slow")
    with pytest.raises(TimeoutError):
        slow.with_timeout(0.05).block_on()
    assert PythonTask(lambda: "fast").with_timeout(5).block_on() == "fast"
    res, idx = PythonTask.select_one([PythonTask(lambda: time.sleep(2) or "a"),
                                      PythonTask(lambda: "b")]).block_on()
    assert (res, idx) == ("b", 1)


def test_shared_is_awaitable_from_asyncio():
    async def main():
        sh = PythonTask.spawn_blocking(lambda: time.sleep(0.05) or 5)
        return await sh + await sh
    assert asyncio.run(main()) == 10


# ------------------------------------------------------------------- endpoint futures
class Slow(Actor):
    @endpoint
    def after(self, delay: float, v: int) -> int:
        time.sleep(delay)
        return v

    @endpoint
    def boom(self):
        raise ValueError("boom")


@pytest.fixture(scope="module")
def slow():
    pm = this_host().spawn_procs(per_host={"gpus": 2})
    yield pm.spawn("slow", Slow)
    pm.stop().get()


def test_awaiting_endpoint_calls_is_event_driven(slow):
    async def main():
        before = N.task_pool_threads()
        futs = [slow.after.call(0.3, i) for i in range(20)]
        t0 = time.monotonic()
        ticks = 0

        async def ticker():
            nonlocal ticks
            while time.monotonic() - t0 < 0.25:
                ticks += 1
                await asyncio.sleep(0.01)
        res = await asyncio.gather(ticker(), *[f._await() for f in futs])
        grown = N.task_pool_threads() - before
        return res[1:], ticks, grown

    res, ticks, grown = asyncio.run(main())
    assert [sorted(v for _, v in vm.items()) for vm in res] == [[i, i] for i in range(20)]
    assert ticks >= 10               # the loop kept running while the calls were pending
    assert grown == 0                # and no pool thread was parked for them


def test_await_surfaces_endpoint_errors_and_plain_futures(slow):
    async def main():
        with pytest.raises(Exception, match="boom"):
            await slow.boom.call()
        return await Future(lambda timeout: time.sleep(0.05) or "plain")
    assert asyncio.run(main()) == "plain"


def test_future_with_timeout_select_and_concurrent_get(slow):
    with pytest.raises(FutureTimeout):
        slow.after.call(1.0, 1).with_timeout(0.05).get()
    assert sorted(v for _, v in slow.after.call(0.0, 3).with_timeout(5).get().items()) == [3, 3]
    a, b = slow.slice(gpus=0).after.call_one(1.0, "a"), slow.slice(gpus=1).after.call_one(0.0, "b")
    assert select_one([a, b], timeout=10) == ("b", 1)
    assert a.get(10) == "a"
    # two threads waiting on one future: one computes, both see the value
    f = slow.after.call(0.2, 9)
    out = []
    ts = [threading.Thread(target=lambda: out.append(f.get(10))) for _ in range(2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    assert len(out) == 2 and all(sorted(v for _, v in o.items()) == [9, 9] for o in out)
    # a wait that times out can be resumed
    g = slow.after.call(0.3, 4)
    with pytest.raises(TimeoutError):
        g.get(0.01)
    assert sorted(v for _, v in g.get(10).items()) == [4, 4]
