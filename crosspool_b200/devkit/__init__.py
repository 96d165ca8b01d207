"""Developer observers: event timelines of the transport / fabric / lane graph / MoE routing, merged
into one chrome-trace file. Every observer is off unless its ``debug.*_observer_enabled`` setting
(or ``XPOOL_DEBUG_*_OBSERVER_ENABLED``) is on, and an un-observed run allocates nothing."""

from .observers import (AtnFabricObserver, FabricObserver, GraphObserver, ObserverSet, RoutingObserver, TransportObserver, chrome_trace,
                        observers_for_role)

__all__ = ["AtnFabricObserver", "FabricObserver", "GraphObserver", "ObserverSet", "RoutingObserver", "TransportObserver", "chrome_trace",
           "observers_for_role"]
