// The number of positions in one page of the key/value cache: the one place it is written.
// The attention kernels tile pages at compile time; the Python side reads this line
// (braidinfer_b200/csrc/build.py: page_size) and the kernels that take the page size as an
// argument are given the same number.
#pragma once
#define BRAID_PAGE_SIZE 64
