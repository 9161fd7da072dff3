"""Router fan-out over the loopback hub and the event router's resend / NACK behaviour."""
import anyio

from exo_b200.routing.event_router import EventRouter
from exo_b200.routing.router import (COMMANDS, CONNECTION_MESSAGES, ELECTION_MESSAGES, GLOBAL_EVENTS, LoopbackHub,
                                     make_router)
from exo_b200.shared.base import NodeId, SessionId, SystemId
from exo_b200.shared.election import ElectionMessage
from exo_b200.shared.events import GlobalForwarderEvent, TestEvent
from exo_b200.shared.messages import ForwarderCommand, RequestEventLog, TestCommand
from exo_b200.utils.channels import channel


def test_router_local_and_network_fanout_and_connection_messages():
    async def main():
        hub = LoopbackHub()
        a, b = NodeId("a"), NodeId("b")
        ra = make_router(a, hub.attach(a))
        rb = make_router(b, hub.attach(b))
        send_a = ra.sender(ELECTION_MESSAGES)
        recv_a, recv_b = ra.receiver(ELECTION_MESSAGES), rb.receiver(ELECTION_MESSAGES)
        conn_a = ra.receiver(CONNECTION_MESSAGES)
        cmd_b = rb.receiver(COMMANDS)
        async with anyio.create_task_group() as tg:
            tg.start_soon(ra.run)
            tg.start_soon(rb.run)
            await anyio.sleep(0.05)
            m = ElectionMessage(clock=1, seniority=0, proposed_session=SessionId(master_node_id=a, election_clock=1), commands_seen=0)
            await send_a.send(m)
            await ra.sender(COMMANDS).send(ForwarderCommand(origin=SystemId("s"), command=TestCommand()))
            await anyio.sleep(0.1)
            assert recv_a.collect() == [m] and recv_b.collect() == [m]
            assert len(cmd_b.collect()) == 1
            ups = conn_a.collect()
            assert ups and ups[0].node_id == b and ups[0].connected
            hub.detach(b)
            await anyio.sleep(0.05)
            downs = conn_a.collect()
            assert downs and not downs[-1].connected
            tg.cancel_scope.cancel()
    anyio.run(main)


def test_event_router_orders_nacks_gaps_and_resends_unechoed_events():
    async def main():
        master = NodeId("m")
        sess = SessionId(master_node_id=master, election_clock=0)
        cmd_s, cmd_r = channel()
        gin_s, gin_r = channel()
        lout_s, lout_r = channel()
        er = EventRouter(sess, cmd_s, gin_r, lout_s, resend_after=0.2, nack_base=0.05)
        out = er.receiver()
        prod = er.sender()
        async with anyio.create_task_group() as tg:
            tg.start_soon(er.run)
            evs = [TestEvent() for _ in range(4)]

            def g(i):
                return GlobalForwarderEvent(origin_idx=i, origin=master, session=sess, event=evs[i])
            await gin_s.send(g(0))
            await gin_s.send(g(2))            # gap at 1
            await gin_s.send(GlobalForwarderEvent(origin_idx=1, origin=NodeId("imposter"), session=sess, event=evs[1]))
            await anyio.sleep(0.2)
            assert [e.idx for e in out.collect()] == [0]
            nacks = cmd_r.collect()
            assert nacks and isinstance(nacks[0].command, RequestEventLog) and nacks[0].command.since_idx == 1
            await gin_s.send(g(1))            # replay closes the gap
            await gin_s.send(g(3))
            await anyio.sleep(0.05)
            assert [e.idx for e in out.collect()] == [1, 2, 3]
            # an event we produced is re-sent until the master echoes it
            mine = TestEvent()
            await prod.send(mine)
            await anyio.sleep(0.7)
            sent = [f for f in lout_r.collect() if f.event.event_id == mine.event_id]
            assert len(sent) >= 2 and all(f.origin_idx == 0 for f in sent)
            await gin_s.send(GlobalForwarderEvent(origin_idx=4, origin=master, session=sess, event=mine))
            await anyio.sleep(0.5)
            assert not er.out_for_delivery and not [f for f in lout_r.collect() if f.event.event_id == mine.event_id]
            tg.cancel_scope.cancel()
    anyio.run(main)
