"""Bully-style master election over the election topic.

Protocol as in the reference (``src/exo/shared/election.py:21-265``): a candidate's ballot is
``(clock, seniority, commands_seen, node id)`` compared in that order; a round starts at boot
(zero time-out), after any connection change (clock + 1, 0.2 s debounce) and whenever a ballot
with a higher clock arrives; when the round's time-out (3 s) expires the greatest ballot wins,
the winner's seniority grows to the number of candidates it beat, and every node emits an
``ElectionResult`` saying whether the session (master, clock) changed.  A non-candidate carries
seniority −1 and can never win against a candidate.

The implementation is one state object with a single "current round" task: starting a round
cancels the previous one, so there is no overlap to reason about.
"""
from __future__ import annotations

from typing import Self

import anyio

from ..utils.channels import ChannelClosed, Receiver, Sender
from .base import FrozenModel, NodeId, SessionId

DEFAULT_ELECTION_TIMEOUT = 3.0
FORCE_MASTER_SENIORITY = 1_000_000


class ElectionMessage(FrozenModel):
    clock: int
    seniority: int
    proposed_session: SessionId
    commands_seen: int

    def _key(self) -> tuple[int, int, int, str]:
        return (self.clock, self.seniority, self.commands_seen, str(self.proposed_session.master_node_id))

    def __lt__(self, other: Self) -> bool:
        return self._key() < other._key()


class ElectionResult(FrozenModel):
    session_id: SessionId
    won_clock: int
    is_new_master: bool


class ConnectionMessage(FrozenModel):
    """A peer appeared on / vanished from the bus (local-only topic)."""
    node_id: NodeId
    connected: bool


class Election:
    def __init__(self, node_id: NodeId, *, election_message_receiver: Receiver[ElectionMessage],
                 election_message_sender: Sender[ElectionMessage], election_result_sender: Sender[ElectionResult],
                 connection_message_receiver: Receiver[ConnectionMessage], command_receiver: Receiver,
                 is_candidate: bool = True, seniority: int = 0, timeout: float = DEFAULT_ELECTION_TIMEOUT):
        self.node_id = node_id
        self.seniority = seniority if is_candidate else -1
        self.clock = 0
        self.commands_seen = 0
        self.timeout = timeout
        self.current_session = SessionId(master_node_id=node_id, election_clock=0)
        self._ballots_in, self._ballots_out = election_message_receiver, election_message_sender
        self._results = election_result_sender
        self._connections, self._commands = connection_message_receiver, command_receiver
        self._round_scope: anyio.CancelScope | None = None
        self._round_candidates: list[ElectionMessage] = []
        self._tg: anyio.abc.TaskGroup | None = None

    # ---- ballots ----
    def ballot(self, clock: int | None = None) -> ElectionMessage:
        c = self.clock if clock is None else clock
        mine = self.current_session.master_node_id == self.node_id
        session = self.current_session if mine else SessionId(master_node_id=self.node_id, election_clock=c)
        return ElectionMessage(clock=c, seniority=self.seniority, proposed_session=session,
                               commands_seen=self.commands_seen)

    async def _announce(self, winner: ElectionMessage) -> None:
        changed = winner.proposed_session != self.current_session
        self.current_session = winner.proposed_session
        await self._results.send(ElectionResult(session_id=winner.proposed_session, won_clock=winner.clock,
                                                is_new_master=changed))

    # ---- one round ----
    def _start_round(self, candidates: list[ElectionMessage], timeout: float) -> None:
        if self._round_scope is not None:
            self._round_scope.cancel()
        self._round_candidates = candidates
        scope = anyio.CancelScope()
        self._round_scope = scope
        assert self._tg is not None
        self._tg.start_soon(self._round, scope, candidates, self.clock, timeout)

    async def _round(self, scope: anyio.CancelScope, candidates: list[ElectionMessage], clock: int, timeout: float) -> None:
        with scope:
            mine = self.ballot(clock)
            candidates.append(mine)
            await self._ballots_out.send(mine)
            await anyio.sleep(timeout)
            await self._ballots_out.send(mine)   # late joiners still see us
            await anyio.sleep(0)
            winner = max(candidates)
            if winner.proposed_session.master_node_id == self.node_id and self.seniority >= 0:
                self.seniority = max(self.seniority, len(candidates))
            if self._round_scope is scope:
                self._round_scope = None
            await self._announce(winner)

    # ---- inputs ----
    async def _on_ballots(self) -> None:
        async for m in self._ballots_in:
            if m.proposed_session.master_node_id == self.node_id:
                continue
            if m.clock > self.clock:
                self.clock = m.clock
                self._start_round([m], self.timeout)
            elif m.clock == self.clock:
                self._round_candidates.append(m)

    async def _on_connections(self) -> None:
        async for _first in self._connections:
            await anyio.sleep(0.2)      # debounce a burst of link changes into one round
            self._connections.collect()
            self.clock += 1
            self._start_round([], self.timeout)

    async def _count_commands(self) -> None:
        async for _ in self._commands:
            self.commands_seen += 1

    async def run(self) -> None:
        try:
            async with anyio.create_task_group() as tg:
                self._tg = tg
                tg.start_soon(self._on_ballots)
                tg.start_soon(self._on_connections)
                tg.start_soon(self._count_commands)
                self._start_round([], 0.0)
        except ChannelClosed:
            pass
        finally:
            self._tg = None

    def shutdown(self) -> None:
        if self._tg is not None:
            self._tg.cancel_scope.cancel()
