// boost::filesystem as used by the engine (path, operator/=, string(),
// create_directories, current_path) is a subset of std::filesystem.
#ifndef LZB_BOOST_SHIM_FILESYSTEM_HPP
#define LZB_BOOST_SHIM_FILESYSTEM_HPP
#include <filesystem>
namespace boost {
namespace filesystem = std::filesystem;
}
#endif
