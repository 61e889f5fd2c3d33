// C interface of the host memory layer (host_memory.cpp), as far as the scheduler uses it.
// Calls return kLsbHostErr on failure; the message is then in lsbm_last_error.
#pragma once
#include <cstdint>

constexpr int kLsbHostErr = -1000;

extern "C" {
const char* lsbm_last_error(void* h);
int lsbm_page_size(void* h);
int lsbm_max_pages(void* h);
int lsbm_smallest_pool(void* h);
int lsbm_open(void* h);
int lsbm_close(void* h, int slot);
long long lsbm_length(void* h, int slot);
int lsbm_num_pages(void* h, int slot);
int lsbm_free_pages(void* h);
int lsbm_reserve(void* h, int slot, long long new_length);
int lsbm_commit(void* h, int slot, long long new_length);
int lsbp_match(void* h, const int* tokens, long long n, int* out, int cap);
long long lsbp_adopt(void* h, int slot, const int* path, int n);
int lsbp_release(void* h, const int* path, int n);
int lsbp_insert(void* h, const int* tokens, long long n, int slot);
int lsbp_share(void* h, const int* tokens, long long n, int slot, const int* held, int n_held, int* added,
               int cap);
int lsbp_evictable(void* h);
int lsbp_evict(void* h, int wanted);
int lsbp_idle_on(void* h, const int* path, int n);
}
