"""Constants and the ctypes "basics" object of the reference's ``collcache.common``
(python/collcache/common/__init__.py), bound to libugache_b200.so."""
import ctypes

from ... import _lib

# cache policy ids (python/collcache/common/__init__.py:46-64 of the reference)
kCacheByDegree, kCacheByHeuristic, kCacheByPreSample, kCacheByDegreeHop = 0, 1, 2, 3
kCacheByPreSampleStatic, kCacheByFakeOptimal, kDynamicCache, kCacheByRandom = 4, 5, 6, 7
kCollCache, kCollCacheIntuitive, kPartitionCache, kPartRepCache, kRepCache = 8, 9, 10, 11, 12
kCollCacheAsymmLink, kCliquePart, kCliquePartByDegree, kSOK, kHPS, kCollFineGrain = 13, 14, 15, 16, 17, 18

cache_policies = {
    'degree': kCacheByDegree, 'heuristic': kCacheByHeuristic, 'pre_sample': kCacheByPreSample,
    'degree_hop': kCacheByDegreeHop, 'presample_static': kCacheByPreSampleStatic,
    'fake_optimal': kCacheByFakeOptimal, 'dynamic_cache': kDynamicCache, 'random': kCacheByRandom,
    'coll_cache': kCollCache, 'coll_intuitive': kCollCacheIntuitive, 'partition': kPartitionCache,
    'part_rep': kPartRepCache, 'rep': kRepCache, 'coll_cache_asymm_link': kCollCacheAsymmLink,
    'coll_fine_grain': kCollFineGrain, 'clique_part': kCliquePart,
    'clique_part_by_degree': kCliquePartByDegree,
}


def cpu(device_id=0):
    return 'cpu:{:}'.format(device_id)


def gpu(device_id=0):
    return 'cuda:{:}'.format(device_id)


# step-log item ids, in the reference's order (python/collcache/common/__init__.py:95-151)
_STEP_ITEMS = [
    "kLogL1NumSample", "kLogL1NumNode", "kLogL1SampleTotalTime", "kLogL1SampleTime",
    "kLogL1SendTime", "kLogL1RecvTime", "kLogL1CopyTime", "kLogL1ConvertTime", "kLogL1TrainTime",
    "kLogL1FeatureBytes", "kLogL1LabelBytes", "kLogL1IdBytes", "kLogL1GraphBytes",
    "kLogL1MissBytes", "kLogL1RemoteBytes", "kLogL1PrefetchAdvanced", "kLogL1GetNeighbourTime",
    "kLogL1SamplerId",
    "kLogL2ShuffleTime", "kLogL2LastLayerTime", "kLogL2LastLayerSize", "kLogL2CoreSampleTime",
    "kLogL2IdRemapTime", "kLogL2GraphCopyTime", "kLogL2IdCopyTime", "kLogL2ExtractTime",
    "kLogL2FeatCopyTime", "kLogL2CacheCopyTime",
    "kLogL3KHopSampleCooTime", "kLogL3KHopSampleKernelTime", "kLogL3KHopSampleSortCooTime",
    "kLogL3KHopSampleCountEdgeTime", "kLogL3KHopSampleCompactEdgesTime",
    "kLogL3RandomWalkSampleCooTime", "kLogL3RandomWalkTopKTime", "kLogL3RandomWalkTopKStep1Time",
    "kLogL3RandomWalkTopKStep2Time", "kLogL3RandomWalkTopKStep3Time",
    "kLogL3RandomWalkTopKStep4Time", "kLogL3RandomWalkTopKStep5Time",
    "kLogL3RandomWalkTopKStep6Time", "kLogL3RandomWalkTopKStep7Time", "kLogL3RemapFillUniqueTime",
    "kLogL3RemapPopulateTime", "kLogL3RemapMapNodeTime", "kLogL3RemapMapEdgeTime",
    "kLogL3CacheGetIndexTime", "KLogL3CacheCopyIndexTime", "kLogL3CacheExtractMissTime",
    "kLogL3CacheCopyMissTime", "kLogL3CacheCombineMissTime", "kLogL3CacheCombineCacheTime",
    "kLogL3CacheCombineRemoteTime", "kLogL3LabelExtractTime",
]
for _i, _n in enumerate(_STEP_ITEMS):
    globals()[_n] = _i


class CollCacheBasics(object):
    """Same methods as the reference's ctypes wrapper
    (python/collcache/common/__init__.py:164-260)."""

    def __init__(self):
        L = _lib.lib()
        self.C_LIB_CTYPES = L
        L.coll_cache_config.argtypes = (ctypes.POINTER(ctypes.c_char_p),
                                        ctypes.POINTER(ctypes.c_char_p), ctypes.c_size_t)
        L.coll_cache_log_step_by_key.argtypes = (ctypes.c_uint64, ctypes.c_int, ctypes.c_double)
        L.coll_cache_report_step_by_key.argtypes = (ctypes.c_uint64,)
        L.coll_cache_report_step_average_by_key.argtypes = (ctypes.c_uint64,)
        L.coll_cache_record_init.argtypes = (ctypes.c_int,)
        L.coll_cache_record.argtypes = (ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t)
        L.coll_cache_lookup.argtypes = (ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                                        ctypes.c_void_p, ctypes.c_void_p)
        L.coll_cache_init_c.argtypes = (ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p,
                                        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int, ctypes.c_size_t, ctypes.c_double,
                                        ctypes.c_void_p)
        L.coll_cache_refresh.argtypes = (ctypes.c_int, ctypes.c_void_p)
        L.coll_cache_set_device.argtypes = (ctypes.c_int, ctypes.c_int)
        L.coll_cache_context.restype = ctypes.c_void_p
        L.coll_cache_wait_one_child.restype = ctypes.c_int
        L.coll_cache_num_epoch.restype = ctypes.c_size_t

    @staticmethod
    def _ok(rc, what):
        if rc != 0:
            raise RuntimeError("%s failed with status %d: %s"
                               % (what, rc, _lib.lib().ugc_last_error().decode()))

    def config(self, run_config: dict):
        keys = [str.encode(str(k)) for k in run_config.keys()]
        vals = []
        for v in run_config.values():
            if isinstance(v, list):
                vals.append(str.encode(' '.join(str(x) for x in v)))
            else:
                vals.append(str.encode(str(v)))
        n = len(keys)
        rc = self.C_LIB_CTYPES.coll_cache_config((ctypes.c_char_p * n)(*keys),
                                                 (ctypes.c_char_p * n)(*vals), n)
        self._ok(rc, "coll_cache_config")

    def log_step_by_key(self, key, item, val):
        return self.C_LIB_CTYPES.coll_cache_log_step_by_key(key, item, val)

    def report_step(self, key):
        return self.C_LIB_CTYPES.coll_cache_report_step_by_key(key)

    def report_step_average(self, key):
        return self.C_LIB_CTYPES.coll_cache_report_step_average_by_key(key)

    def train_barrier(self):
        self._ok(self.C_LIB_CTYPES.coll_cache_train_barrier(), "coll_cache_train_barrier")

    def wait_one_child(self):
        return self.C_LIB_CTYPES.coll_cache_wait_one_child()

    def print_memory_usage(self):
        return self.C_LIB_CTYPES.coll_cache_print_memory_usage()

    def coll_cache_record_init(self, replica_id):
        self._ok(self.C_LIB_CTYPES.coll_cache_record_init(replica_id), "coll_cache_record_init")

    def shutdown(self):
        self.C_LIB_CTYPES.coll_cache_shutdown()


_basics = CollCacheBasics()
