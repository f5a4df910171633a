"""CPU side of serving: KV page accounting, request records, trace frontend, batch scheduler."""
from .kv_cache import DistKVPool, DistKVCache, BatchedDistKVCache, KVPoolExhausted
from .request import NewRequestInfo, NewRequestQueue, FlyRequestInfo
from .frontend import RequestManager, requestManager
from .scheduler import Scheduler, BatchPlan, WorkingSet
