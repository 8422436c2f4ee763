// Host-initiated atomics on symmetric objects.  The operation itself is one
// atom.sys issued by a one-thread kernel on the internal stream (or a C++ atomic
// on the host-memory heap); the old value comes back through pinned memory.
#pragma once
#include <cstddef>
namespace bshmem {
enum AmoOp { AMO_ADD = 0, AMO_FETCH_ADD, AMO_CAS, AMO_SWAP, AMO_FETCH, AMO_AND, AMO_OR, AMO_XOR };
// `width` is 4 or 8 bytes; `value`/`cond` point to operands of that width; `old`
// (optional) receives the previous contents.  Returns a Status.
int host_amo(int op, void* target, const void* value, const void* cond, size_t width, int pe, void* old);
}  // namespace bshmem
