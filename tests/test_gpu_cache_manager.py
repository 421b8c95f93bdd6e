"""GetCacheLocation / StartWriteCache / FinishWriteCache over a device-resident index, replaying the reference's own
CacheManager tests (kv_cache_manager/manager/test/cache_manager_test.cc:464-905): same calls in the same order, the
counts and the empty / non-empty locations they assert.  Where the reference returns CacheLocation objects this
returns one bool per location (True = it carries a URI)."""
import numpy as np
import pytest

from oracle import kvcm_oracle as oracle

import tair_kvcache_b200  # noqa: F401
from tair_kvcache_b200.manager import GpuCacheManager, QueryType
from tair_kvcache_b200.manager import cache_manager as cm

pytestmark = pytest.mark.gpu
PREFIX, BATCH_GET, SW = QueryType.QT_PREFIX_MATCH, QueryType.QT_BATCH_GET, QueryType.QT_REVERSE_ROLL_SW_MATCH


def _manager():
    m = GpuCacheManager("cuda:0")
    assert m.RegisterInstance("test_instance", 64, 4096) == cm.EC_OK
    return m


def test_prefix_match_flow():  # TestGetCacheLocationPrefixMatch, :464-545
    m = _manager()
    keys = [1, 2, 3]
    ec, session, mask, n_new = m.StartWriteCache("test_instance", keys)
    assert (ec, mask, n_new) == (cm.EC_OK, 0, 3)
    ec, loc = m.GetCacheLocation("test_instance", PREFIX, keys)
    assert ec == cm.EC_OK and len(loc) == 0           # written, not served yet
    assert m.FinishWriteCache("test_instance", session, 3) == cm.EC_OK
    assert len(m.GetCacheLocation("test_instance", PREFIX, keys)[1]) == 3
    assert len(m.GetCacheLocation("test_instance", PREFIX, [1, 2, 4, 3])[1]) == 2
    assert len(m.GetCacheLocation("test_instance", PREFIX, [1, 2, 3, 12212])[1]) == 3   # TestGetCacheNotExistLocation
    # a session finishes once (:440-460: the second finish finds no session)
    assert m.FinishWriteCache("test_instance", session, 3) == cm.EC_ERROR


def test_batch_get_flow():  # TestGetCacheLocationBatchGet, :547-630
    m = _manager()
    ec, session, mask, n_new = m.StartWriteCache("test_instance", [1, 2, 3, 4])
    assert ec == cm.EC_OK
    ec, loc = m.GetCacheLocation("test_instance", BATCH_GET, [1, 2, 3, 4])
    assert ec == cm.EC_OK and len(loc) == 4
    assert m.FinishWriteCache("test_instance", session, 3) == cm.EC_OK
    assert m.GetCacheLocation("test_instance", BATCH_GET, [1, 2, 3, 4])[1].tolist() == [True, True, True, False]
    assert m.GetCacheLocation("test_instance", BATCH_GET, [1, 2, 111, 4])[1].tolist() == [True, True, False, False]


def test_reverse_roll_sliding_window_flow():  # TestGetCacheLocationReverseRollSlideWindowMatch, :632-750
    m = _manager()
    keys = [1, 2, 3, 4, 5, 6]
    ec, session, _, _ = m.StartWriteCache("test_instance", keys)
    ec, loc = m.GetCacheLocation("test_instance", SW, keys, sw_size=2)
    assert ec == cm.EC_OK and loc.tolist() == [False] * 6
    assert m.FinishWriteCache("test_instance", session, 5) == cm.EC_OK
    assert len(m.GetCacheLocation("test_instance", SW, keys, sw_size=3)[1]) == 6
    got = m.GetCacheLocation("test_instance", SW, [1, 2, 3, 4, 5, 6, 7], sw_size=2)[1]
    assert got.tolist() == [False, False, False, True, True, False, False]
    got = m.GetCacheLocation("test_instance", SW, [1, 2, 3, 10, 5, 6, 7], sw_size=2)[1]
    assert got.tolist() == [False, True, True, False, False, False, False]
    assert m.GetCacheLocation("test_instance", SW, [1], sw_size=2)[0] == cm.EC_BADARGS     # cache_manager.cc:991-994
    assert m.GetCacheLocation("test_instance", SW, [1], sw_size=-1)[0] == cm.EC_BADARGS


def test_finish_write_cache_with_block_masks():  # TestFinishWriteCacheWithBlockMask, :786-905
    m = _manager()
    keys = [1, 2, 3]
    ec, session, _, _ = m.StartWriteCache("test_instance", keys)
    assert len(m.GetCacheLocation("test_instance", PREFIX, keys)[1]) == 0
    assert m.FinishWriteCache("test_instance", session, 2) == cm.EC_OK
    assert len(m.GetCacheLocation("test_instance", PREFIX, keys)[1]) == 2
    # the failed block's location is gone (the reference: CLS_DELETING on its way to CLS_NOT_FOUND)
    assert m.GetCacheLocation("test_instance", BATCH_GET, keys)[1].tolist() == [True, True, False]
    keys = [4, 5, 6, 7]
    ec, session, _, _ = m.StartWriteCache("test_instance", keys)
    assert len(m.GetCacheLocation("test_instance", PREFIX, keys)[1]) == 0
    assert m.FinishWriteCache("test_instance", session, [True, True, False, True]) == cm.EC_OK
    assert len(m.GetCacheLocation("test_instance", PREFIX, keys)[1]) == 2
    assert m.GetCacheLocation("test_instance", BATCH_GET, keys)[1].tolist() == [True, True, False, True]
    # an invalid mask: a vector of another length, an offset beyond the session's keys (cache_location.cc:22-31)
    ec, session, _, _ = m.StartWriteCache("test_instance", [8, 9])
    assert m.FinishWriteCache("test_instance", session, [True]) == cm.EC_BADARGS
    ec, session, _, _ = m.StartWriteCache("test_instance", [10, 11])
    assert m.FinishWriteCache("test_instance", session, 3) == cm.EC_BADARGS


def test_start_write_filters_what_is_there():
    """FilterWriteCache inside StartWriteCache (cache_manager.cc:589-635): a second write of a longer request gets
    the offset of the first missing key; holes give the vector form, and only the holes are written."""
    m = _manager()
    ec, s1, mask, n_new = m.StartWriteCache("test_instance", [1, 2, 3])
    assert m.FinishWriteCache("test_instance", s1, 3) == cm.EC_OK
    ec, s2, mask, n_new = m.StartWriteCache("test_instance", [1, 2, 3, 4, 5])
    assert (ec, mask, n_new) == (cm.EC_OK, 3, 2)
    # still being written: another writer of the same keys has nothing to do (they exist for write)
    ec, s3, mask, n_new = m.StartWriteCache("test_instance", [1, 2, 3, 4, 5])
    assert (mask, n_new) == (5, 0) and m.FinishWriteCache("test_instance", s3, 0) == cm.EC_OK
    assert m.FinishWriteCache("test_instance", s2, [True, False]) == cm.EC_OK     # 4 served, 5 failed and removed
    ec, s4, mask, n_new = m.StartWriteCache("test_instance", [1, 9, 3, 5, 4])
    assert mask == [True, False, True, False, True] and n_new == 2
    assert m.FinishWriteCache("test_instance", s4, 2) == cm.EC_OK
    assert len(m.GetCacheLocation("test_instance", PREFIX, [1, 9, 3, 5, 4])[1]) == 5
    # errors of CheckInputAndGetMetaSearcher (:906-924)
    assert m.StartWriteCache("nobody", [1])[0] == cm.EC_INSTANCE_NOT_EXIST
    assert m.GetCacheLocation("test_instance", PREFIX, [], [])[0] == cm.EC_BADARGS
    assert m.GetCacheLocation("test_instance", QueryType.QT_UNSPECIFIED, [1])[0] == cm.EC_ERROR


def test_tokens_instead_of_keys():
    """Requests that carry token ids are hashed first (GenKeyVector over the instance's block size, :311-314)."""
    m = _manager()
    rng = np.random.default_rng(3)
    toks = rng.integers(0, 151936, size=64 * 5 + 17)
    ec, session, mask, n_new = m.StartWriteCache("test_instance", tokens=toks)
    assert (ec, mask, n_new) == (cm.EC_OK, 0, 5)
    assert m.FinishWriteCache("test_instance", session, 5) == cm.EC_OK
    want = oracle.gen_key_vector(toks.astype(np.int64), 64)
    assert len(m.GetCacheLocation("test_instance", PREFIX, keys=want.tolist())[1]) == 5
    other = toks.copy()
    other[64 * 3 + 1] += 1
    assert len(m.GetCacheLocation("test_instance", PREFIX, tokens=other)[1]) == 3
    assert len(m.GetCacheLocation("test_instance", PREFIX, tokens=toks, block_mask=2)[1]) == 3   # two skipped, three found


def test_remove_and_trim():
    m = _manager()
    ec, session, _, _ = m.StartWriteCache("test_instance", [1, 2, 3, 4])
    assert m.FinishWriteCache("test_instance", session, 4) == cm.EC_OK
    assert m.RemoveCache("test_instance", [3]) == cm.EC_OK
    assert m.GetCacheLocation("test_instance", BATCH_GET, [1, 2, 3, 4])[1].tolist() == [True, True, False, True]
    assert len(m.GetCacheLocation("test_instance", PREFIX, [1, 2, 3, 4])[1]) == 2
    assert m.RemoveCache("test_instance", [], []) == cm.EC_BADARGS and m.RemoveCache("nobody", [1]) == cm.EC_INSTANCE_NOT_EXIST
    assert m.TrimCache("test_instance") == cm.EC_OK and m.index_of("test_instance").stats()[1] == 0
    assert len(m.GetCacheLocation("test_instance", PREFIX, [1, 2])[1]) == 0
    assert m.TrimCache("test_instance", remove_all=False) == cm.EC_OK + 1007


def test_write_session_times_out():  # TestWriteCacheTimeout, cache_manager_test.cc:437-461
    import time
    m = _manager()
    keys = [1, 2]
    ec, session, mask, n_new = m.StartWriteCache("test_instance", keys, write_timeout_seconds=1)
    assert (ec, mask, n_new) == (cm.EC_OK, 0, 2)
    assert m.ExpireWriteSessions(now=time.monotonic() + 0.5) == 0        # not yet
    assert m.ExpireWriteSessions(now=time.monotonic() + 6.0) == 1        # the reference's test sleeps six seconds
    assert m.FinishWriteCache("test_instance", session, 2) == cm.EC_ERROR
    assert m.GetCacheLocation("test_instance", BATCH_GET, keys)[1].tolist() == [False, False]
    assert m.index_of("test_instance").stats()[1] == 0                   # the half-written locations are gone
